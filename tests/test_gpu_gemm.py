"""Batched decode + GEMM entry points vs the oracle."""
import numpy as np
import pytest
import torch

from gpu_util import REL_TOL, assert_close, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from turbo_lossless_b200 import Split12Engine
    return Split12Engine()


def _cw(p, **kw):
    from turbo_lossless_b200 import CompressedWeight
    return CompressedWeight.from_packed(p, **kw)


def _case(O, M, K, B, seed, frac=1e-3):
    w = O.synth_weights(M, K, seed, outlier_frac=frac)
    return w, O.pack(w), O.synth_acts(B, K, seed)


@pytest.mark.parametrize("B", [1, 2, 16, 17, 48, 64, 128, 256])
@pytest.mark.parametrize("M,K", [(128, 256), (200, 512), (4096, 4096), (1024, 4096)])
def test_legacy_gemm_two_pass(eng, O, M, K, B):
    """nv_launch_split12_fused_gemm_async with null patch pointers (what the engine passes), then
    nv_launch_patches_batch_async on the non-empty rows: the reference's batched two passes."""
    w, p, x = _case(O, M, K, B, B + M)
    cw, xd = _cw(p), dev(x)
    out = torch.full((B, M), float("nan"), device="cuda")
    eng.gemm_only(cw, xd, out, K, M, B)
    assert_close(out, O.gemm_twopass(p, x, patches=False), what="first pass")
    eng.patches_batch(cw, xd, out, K, M, B)
    assert_close(out, O.gemm_twopass(p, x), what="two pass")


@pytest.mark.parametrize("B", [16, 48, 64, 256])
def test_v3_and_cublas_entry_points(eng, O, B):
    M, K = 256, 1024
    w, p, x = _case(O, M, K, B, 7)
    cw, xd = _cw(p), dev(x)
    ref = O.gemm_twopass(p, x, patches=False)
    out = torch.empty((B, M), device="cuda")
    eng.gemm_only(cw, xd, out, K, M, B, v3=True)
    assert_close(out, ref, what="v3")
    out.fill_(float("nan"))
    eng.gemm_cublas_path(cw, xd, out, K, M, B)
    assert_close(out, ref, what="cublas-path entry point")


@pytest.mark.parametrize("B", [24, 64, 100, 256])
@pytest.mark.parametrize("M,K", [(128, 256), (130, 320), (4096, 4096)])
def test_fused_exact_with_strides(eng, O, M, K, B):
    w, p, x = _case(O, M, K, B, 3 * B + M, frac=2e-3)
    act_stride, out_stride = K + 64, M + 8
    xd = torch.zeros((B, act_stride), dtype=torch.int16, device="cuda")
    xd[:, :K] = dev(x)
    out = torch.full((B, out_stride), float("nan"), device="cuda")
    eng.gemm(_cw(p), xd, out, act_stride, out_stride, B)
    assert_close(out[:, :M], O.gemm_exact(w, x), what="fused gemm")
    assert torch.isnan(out[:, M:]).all()
    # the legacy name with all four patch pointers given is exact too
    out2 = torch.empty((B, out_stride), device="cuda")
    eng.gemm_only(_cw(p), xd, out2, act_stride, out_stride, B, patched=True)
    assert_close(out2[:, :M], O.gemm_exact(w, x), what="legacy gemm with patch pointers")


def test_zero_batch_and_bad_strides(eng, O):
    w, p, x = _case(O, 128, 256, 4, 1)
    cw, xd = _cw(p), dev(x)
    out = torch.empty((4, 128), device="cuda")
    lib = eng.lib
    args = (cw.split_sm.data_ptr(), cw.split_gr.data_ptr(), p.base_exp, xd.data_ptr())
    assert lib.nv_launch_split12_fused_gemm_async(*args, 256, out.data_ptr(), 128, 128, 256, 0, None,
                                                  None, None, None, None) == 0
    assert lib.nv_launch_split12_fused_gemm_async(*args, 100, out.data_ptr(), 128, 128, 256, 4, None,
                                                  None, None, None, None) < 0


@pytest.mark.parametrize("B", [24, 64, 256])
def test_multi_tensor_launch_qkv(eng, O, B):
    """q/k/v-like tensors (own base_exp, own row counts, one with a ragged row count) in one launch."""
    K = 1024
    specs = [(512, 0.02, 1e-3), (130, 0.05, 5e-3), (128, 0.01, 0.0)]
    ws, packs = [], []
    for i, (M, std, frac) in enumerate(specs):
        w = O.synth_weights(M, K, 200 + i, std=std, outlier_frac=frac)
        ws.append(w); packs.append(O.pack(w))
    x = O.synth_acts(B, K, 9)
    xd = dev(x)
    outs = [torch.full((B, p.M + 4), float("nan"), device="cuda") for p in packs]
    eng.gemm_multi([_cw(p) for p in packs], xd, outs, K, B)
    for w, p, o in zip(ws, packs, outs):
        assert_close(o[:, :p.M], O.gemm_exact(w, x), what=f"M={p.M}")
        assert torch.isnan(o[:, p.M:]).all()
    assert eng.device_status() == 0


@pytest.mark.parametrize("knobs", [{"S12_GEMM_CLUSTER": "0", "S12_GEMM_SPLIT": "0"},      # stream-K with owner hand-over
                                   {"S12_GEMM_CLUSTER": "0", "S12_GEMM_SPLIT": "1"},      # whole tiles
                                   {"S12_GEMM_CLUSTER": "0", "S12_GEMM_SPLIT": "3"},      # fixed parts, hand-over through the workspace
                                   {"S12_GEMM_CLUSTER": "2"}, {"S12_GEMM_CLUSTER": "5"}, {"S12_GEMM_CLUSTER": "8"},
                                   {}])                                                    # the library's own choice
@pytest.mark.parametrize("M,K,B", [(1000, 4096, 256), (3000, 2048, 100), (20000, 1024, 48)])
def test_every_schedule_gives_the_oracle_result(eng, O, monkeypatch, knobs, M, K, B):
    """The tensor-core GEMM's schedules (stream-K, whole tiles, fixed K parts, clusters of 2..8 CTAs per tile) are
    selected by a cost model; the tuning knobs force each of them here.  Two runs of a schedule are bit-identical."""
    for k, v in knobs.items():
        monkeypatch.setenv(k, v)
    w, p, x = _case(O, M, K, B, M + B, frac=2e-3)
    cw = _cw(p)
    xd = torch.from_numpy(x.view(np.int16)).cuda()
    outs = []
    for _ in range(2):
        out = torch.full((B, M), float("nan"), device="cuda")
        eng.gemm(cw, xd, out, K, M, B)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy())
    assert eng.device_status() == 0
    ref = O.gemm_exact(w, x)
    assert np.abs(outs[0] - ref).max() <= REL_TOL * np.abs(ref).max()
    np.testing.assert_array_equal(outs[0], outs[1])


def _tiled(O, p, tiles):
    """`tiles` copies of a packed slab stacked into one tall tensor (CSR offsets shifted per copy)."""
    ro = np.concatenate([[0]] + [p.row_off[1:].astype(np.int64) + t * p.num_patches for t in range(tiles)])
    return O.Packed(p.M * tiles, p.K, p.base_exp, np.tile(p.sm, tiles), np.tile(p.gr, tiles), ro.astype(np.int32),
                    np.tile(p.cols, tiles), np.tile(p.correct, tiles), np.tile(p.wrong, tiles))


@pytest.mark.parametrize("rows,tiles,K,B", [(4096, 1, 14336, 256),      # down projection: 56 raw stages per tile
                                            (4008, 32, 4096, 256),      # lm_head 128256 x 4096: 1002 tiles, many per CTA
                                            (4096, 1, 4096, 128),
                                            (1024, 1, 8192, 64),        # 70B k/v projection
                                            (512, 1, 28672, 64)])       # 70B down projection (K = 28672)
def test_benchmark_shapes(eng, O, rows, tiles, K, B):
    """The largest launches of the B=256 and 70B benchmarks.  The oracle packs one slab of `rows` rows; the
    device tensor is `tiles` copies of it, so every copy's output block must equal the slab's oracle result."""
    w = O.synth_weights(rows, K, rows + K + B, outlier_frac=5e-4)
    p = O.pack(w)
    x = O.synth_acts(B, K, 21)
    big = _tiled(O, p, tiles) if tiles > 1 else p
    M = rows * tiles
    out = torch.full((B, M), float("nan"), device="cuda")
    eng.gemm(_cw(big, escape_table=False), dev(x), out, K, M, B)
    assert eng.device_status() == 0
    ref = O.gemm_exact(w, x)
    got = out.cpu().numpy()
    for t in range(tiles):
        assert_close(got[:, t * rows:(t + 1) * rows], ref, what=f"copy {t}")


def _tiny_exponent_weights(M, K, seed, escapes):
    """bf16 patterns whose exponent fields lie in 1..14 (plus exact zeros), so that the packer's window starts at
    exponent 0 and base_exp is -1; `escapes` adds a few values above the window."""
    rng = np.random.default_rng(seed)
    w = ((rng.integers(0, 2, (M, K)) << 15) | (rng.integers(1, 15, (M, K)) << 7) | rng.integers(0, 128, (M, K))).astype(np.uint16)
    w[rng.random((M, K)) < 0.02] = 0
    if escapes:
        mask = rng.random((M, K)) < 2e-3
        w[mask] = ((rng.integers(15, 19, (M, K)) << 7) | rng.integers(0, 128, (M, K))).astype(np.uint16)[mask]
    return w


@pytest.mark.parametrize("B", [24, 256])
@pytest.mark.parametrize("escapes", [False, True])
def test_window_starting_at_exponent_zero(eng, O, B, escapes):
    """base_exp = -1 (split12_pack.c:29-35) through the batched kernels: exact with the CSR list; without it
    escapes keep the reference's bits (exponent field 0xFF: infinities and NaNs in their rows)."""
    M, K = 300, 512
    w = _tiny_exponent_weights(M, K, 5 + B, escapes)
    p = O.pack(w)
    assert p.base_exp == -1 and (p.num_patches > 0) == escapes
    x = (O.synth_acts(B, K, 4) + np.uint16(100 << 7)).astype(np.uint16)      # activations * 2^100: products are normal fp32
    xd = dev(x)
    out = torch.full((B, M), float("nan"), device="cuda")
    eng.gemm(_cw(p), xd, out, K, M, B)
    assert_close(out, O.gemm_exact(w, x), what="with the CSR list")
    out2 = torch.full((B, M), float("nan"), device="cuda")
    eng.gemm_only(_cw(p), xd, out2, K, M, B)                                  # null patch pointers
    ref = O.gemm_twopass(p, x, patches=False)
    got = out2.cpu().numpy()
    fin = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), fin)
    if escapes:
        assert not fin.all()
    scale = np.abs(ref[fin]).max()
    assert np.abs(got[fin] - ref[fin]).max() <= REL_TOL * scale
    assert eng.device_status() == 0


@pytest.mark.parametrize("knobs", [{}, {"S12_GEMM_CLUSTER": "0", "S12_GEMM_SPLIT": "0"}, {"S12_GEMM_CLUSTER": "2"}])
@pytest.mark.parametrize("B", [257, 300, 512])
def test_more_than_one_tile_of_sequences(eng, O, monkeypatch, knobs, B):
    """B > 256: several sequence tiles per row tile (tile -> (row tile, sequence tile) decomposition, drain
    offsets, stream-K ownership across sequence tiles), on the default, stream-K and cluster schedules."""
    for k, v in knobs.items():
        monkeypatch.setenv(k, v)
    M, K = 700, 1024
    w, p, x = _case(O, M, K, B, B, frac=2e-3)
    out = torch.full((B, M + 4), float("nan"), device="cuda")
    eng.gemm(_cw(p), dev(x), out, K, M + 4, B)
    assert_close(out[:, :M], O.gemm_exact(w, x), what=f"B={B}")
    assert torch.isnan(out[:, M:]).all()
    assert eng.device_status() == 0


def test_grouped_launch_with_several_sequence_tiles(eng, O):
    K, B = 512, 300
    specs = [(256, 0), (130, 300), (384, 0)]                 # (rows, first activation row)
    x = O.synth_acts(2 * B, K, 31)
    ws, cws = [], []
    for i, (M, _) in enumerate(specs):
        w = O.synth_weights(M, K, 300 + i, outlier_frac=1e-3)
        ws.append(w); cws.append(_cw(O.pack(w)))
    outs = [torch.full((B, M), float("nan"), device="cuda") for M, _ in specs]
    eng.gemm_grouped(cws, dev(x), [r0 for _, r0 in specs], outs, K, B)
    for w, (M, r0), o in zip(ws, specs, outs):
        assert_close(o, O.gemm_exact(w, x[r0:r0 + B]), what=f"M={M} rows from {r0}")
    assert eng.device_status() == 0
