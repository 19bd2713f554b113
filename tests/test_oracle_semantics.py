"""Oracle GEMV/GEMM semantics, the escape table and the tensor-parallel sharder (CPU only)."""
import numpy as np
import pytest


def _case(O, M, K, seed, frac=5e-3):
    w = O.synth_weights(M, K, seed, outlier_frac=frac)
    return w, O.pack(w)


def test_twopass_equals_exact_up_to_rounding(O):
    w, p = _case(O, 96, 512, 11)
    x = O.synth_acts(5, 512, 11)
    two, ex = O.gemm_twopass(p, x), O.gemm_exact(w, x)
    assert two.shape == (5, 96)
    assert np.max(np.abs(two - ex)) <= 1e-5 * np.max(np.abs(ex))
    # without the second pass the escapes matter
    first = O.gemm_twopass(p, x, patches=False)
    assert np.max(np.abs(first - ex)) > 1e-3 * np.max(np.abs(ex))
    # first pass == exact GEMM on the "wrong" unpack
    assert np.allclose(first, O.gemm_exact(O.unpack_wrong(p), x), rtol=0, atol=1e-6 * np.max(np.abs(ex)))


def test_cpu_baseline_matches_checker(O):
    w, p = _case(O, 64, 1024, 12)
    x = O.synth_acts(3, 1024, 12)
    got, ex = O.cpu_unpack_gemm_f32(p, x), O.gemm_exact(w, x)
    assert np.max(np.abs(got - ex)) <= 1e-5 * np.max(np.abs(ex))


def test_escape_table_order(O):
    """(row, col mod 256, ascending col) order, row_base = exclusive row prefix (model.cpp:92-125)."""
    w, p = _case(O, 40, 1024, 13, frac=2e-2)
    row_base, counts, vals, nonempty = O.build_escape_table(p)
    assert np.array_equal(row_base, p.row_off[:-1])
    exp_vals, exp_ne = [], []
    for r in range(p.M):
        lo, hi = p.row_off[r], p.row_off[r + 1]
        if hi > lo:
            exp_ne.append(r)
        c = p.cols[lo:hi]
        order = np.lexsort((c, c % 256))
        exp_vals.extend(p.correct[lo:hi][order])
        cnt = np.bincount(c % 256, minlength=256)
        assert np.array_equal(counts[r * 256:(r + 1) * 256], cnt.astype(np.uint8))
    assert np.array_equal(vals, np.array(exp_vals, np.int16))
    assert np.array_equal(nonempty, np.array(exp_ne, np.int32))


@pytest.mark.parametrize("parts", [2, 4, 8])
def test_row_and_col_shards_decode_to_slices(O, parts):
    w, p = _case(O, 64, 512, 14, frac=1e-2)
    for i in range(parts):
        r0, r1 = i * p.M // parts, (i + 1) * p.M // parts
        s = O.shard_rows(p, r0, r1)
        assert s.base_exp == p.base_exp
        assert np.array_equal(O.unpack_exact(s), w[r0:r1])
        c0, c1 = i * p.K // parts, (i + 1) * p.K // parts
        s = O.shard_cols(p, c0, c1)
        assert np.array_equal(O.unpack_exact(s), w[:, c0:c1])
        assert np.array_equal(O.unpack_wrong(s), O.unpack_wrong(p)[:, c0:c1])


def test_row_parallel_partials_sum_to_full(O):
    w, p = _case(O, 48, 1024, 15)
    x = O.synth_acts(2, 1024, 15)
    full = O.gemm_twopass(p, x).astype(np.float64)
    acc = np.zeros_like(full)
    for i in range(4):
        c0, c1 = i * 256, (i + 1) * 256
        acc += O.gemm_twopass(O.shard_cols(p, c0, c1), x[:, c0:c1])
    assert np.max(np.abs(acc - full)) <= 1e-5 * np.max(np.abs(full))
