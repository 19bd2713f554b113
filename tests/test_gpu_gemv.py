"""Decode + GEMV family vs the oracle, through the drop-in entry points and the fused ones."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, golden_packed
from gpu_util import assert_close, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from turbo_lossless_b200 import Split12Engine
    return Split12Engine()


def _cw(p, **kw):
    from turbo_lossless_b200 import CompressedWeight
    return CompressedWeight.from_packed(p, **kw)


def _case(O, M, K, seed, frac=5e-4, B=1):
    w = O.synth_weights(M, K, seed, outlier_frac=frac)
    p = O.pack(w)
    x = O.synth_acts(B, K, seed)
    return w, p, x


SHAPES = [(16, 128), (1, 32), (2, 64), (15, 96), (17, 160), (130, 256), (64, 4096), (33, 14336),
          (4096, 4096), (1024, 4096), (1000, 1056), (257, 11008), (4099, 4096), (2050, 14336),
          # Llama-3-70B row lengths: K = 8192 (two CTAs per SM) and K = 28672, whose activation vector leaves
          # room for one CTA per SM only in the streaming kernel
          (64, 8192), (1000, 8192), (64, 28672), (1000, 28672)]


@pytest.mark.parametrize("M,K", SHAPES)
def test_legacy_two_pass_b1(eng, O, M, K):
    """nv_launch_split12_v2_async then nv_launch_patches_async == the reference's two passes."""
    w, p, x = _case(O, M, K, M * 7 + K, frac=2e-3)
    cw, xd = _cw(p), dev(x[0])
    out = torch.full((M,), float("nan"), device="cuda")
    eng.matvec_b1_nopatch(cw, xd, out)
    assert_close(out, O.gemm_twopass(p, x, patches=False)[0], what="first pass")
    eng.patches(cw, xd, out)
    assert_close(out, O.gemm_twopass(p, x)[0], what="two pass")
    # portable twins
    out2 = torch.empty_like(out)
    eng.matvec_b1_nopatch(cw, xd, out2, portable=True)
    eng.patches(cw, xd, out2, portable=True)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("M,K", [(16, 128), (130, 256), (14336, 4096), (1000, 8192)])
def test_legacy_dual(eng, O, M, K):
    wa, pa, x = _case(O, M, K, 31, frac=1e-3)
    wb = O.synth_weights(M, K, 32, std=0.05)
    pb = O.pack(wb)
    assert pa.base_exp != pb.base_exp or M < 100
    ca, cb, xd = _cw(pa), _cw(pb), dev(x[0])
    oa, ob = torch.empty(M, device="cuda"), torch.empty(M, device="cuda")
    eng.matvec_dual(ca, cb, xd, oa, ob)
    assert_close(oa, O.gemm_twopass(pa, x, patches=False)[0], what="dual a")
    assert_close(ob, O.gemm_twopass(pb, x, patches=False)[0], what="dual b")
    eng.patches_b1_batched([(ca, xd, oa), (cb, xd, ob)])
    assert_close(oa, O.gemm_twopass(pa, x)[0], what="dual a patched")
    assert_close(ob, O.gemm_twopass(pb, x)[0], what="dual b patched")


@pytest.mark.parametrize("M,K", SHAPES)
def test_fused_exact_b1(eng, O, M, K):
    w, p, x = _case(O, M, K, M + K * 3, frac=2e-3)
    out = torch.full((M,), float("nan"), device="cuda")
    eng.gemv([_cw(p)], dev(x[0]), [out])
    assert_close(out, O.gemm_exact(w, x)[0], what="fused")


@pytest.mark.parametrize("R", [2, 4, 8, 16])
@pytest.mark.parametrize("depth", [2, 8])
@pytest.mark.parametrize("M,K", [(50, 128), (37, 1056), (300, 4096), (70, 9248)])
def test_streaming_kernel_tilings(eng, O, monkeypatch, R, depth, M, K):
    """The persistent streaming kernel with every rows-per-tile setting and a shallow/deep ring,
    forced on for small shapes (tuning knobs read from the environment at each call)."""
    monkeypatch.setenv("S12_GEMV_IMPL", "2")
    monkeypatch.setenv("S12_GEMV_R", str(R))
    monkeypatch.setenv("S12_GEMV_DEPTH", str(depth))
    w, p, x = _case(O, M, K, R * 100 + M, frac=5e-3)
    out = torch.full((M,), float("nan"), device="cuda")
    eng.gemv([_cw(p)], dev(x[0]), [out])
    assert_close(out, O.gemm_exact(w, x)[0], what=f"R={R} depth={depth}")
    assert eng.device_status() == 0


def test_register_kernel_still_selectable(eng, O, monkeypatch):
    monkeypatch.setenv("S12_GEMV_IMPL", "0")
    w, p, x = _case(O, 4096, 4096, 5)
    out = torch.empty(4096, device="cuda")
    eng.gemv([_cw(p)], dev(x[0]), [out])
    assert_close(out, O.gemm_exact(w, x)[0])


def test_fused_qkv_one_launch(eng, O):
    K = 4096
    packs = [O.pack(O.synth_weights(M, K, 40 + i, outlier_frac=1e-3)) for i, M in enumerate((4096, 1024, 1000))]
    x = O.synth_acts(1, K, 44)
    outs = [torch.empty(p.M, device="cuda") for p in packs]
    eng.gemv([_cw(p) for p in packs], dev(x[0]), outs)
    for p, o in zip(packs, outs):
        assert_close(o, O.gemm_twopass(p, x)[0], what=f"qkv M={p.M}")


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_cases(eng, O, golden, name):
    """Includes K=130 (general path), all-escape rows and base_exp = -1."""
    w, p = golden_packed(O, golden, name)
    x = O.synth_acts(1, p.K, 3)
    if name == "wide_exponents_16x128":
        x = x - np.uint16(40 << 7)                   # activations * 2^-40: keeps fp32 sums finite
    out = torch.empty(p.M, device="cuda")
    eng.gemv([_cw(p)], dev(x[0]), [out])
    wf = O.bf16_bits_to_f32(w)
    if not np.all(np.isfinite(wf)):                  # inf/nan weights: compare against numpy directly
        ref = (wf.astype(np.float64) @ O.bf16_bits_to_f32(x[0]).astype(np.float64))
        got = out.cpu().numpy()
        fin = np.isfinite(ref)
        assert np.array_equal(np.isnan(got), np.isnan(ref))
        assert np.allclose(got[fin], ref[fin], rtol=1e-4, atol=1e-4 * np.max(np.abs(ref[fin]) + 1e-30))
        return
    ref = O.gemm_exact(w, x)[0]
    if name == "wide_exponents_16x128":              # exponents up to 2^127: scale by the abs-sum
        bound = O.gemm_abs(w, x)[0]
        assert np.all(np.abs(out.cpu().numpy() - ref) <= 1e-4 * bound)
    else:
        assert_close(out, ref, what=name)


@pytest.mark.parametrize("B", [2, 3, 4, 8, 9, 16])
@pytest.mark.parametrize("M,K", [(16, 128), (130, 256), (100, 4096), (4096, 4096)])
def test_fused_small_batch(eng, O, M, K, B):
    w, p, x = _case(O, M, K, 50 + B, frac=2e-3, B=B)
    act_stride, out_stride = K + 64, M + 3
    xd = torch.zeros((B, act_stride), dtype=torch.int16, device="cuda")
    xd[:, :K] = dev(x)
    out = torch.full((B, out_stride), float("nan"), device="cuda")
    eng.gemv_batched(_cw(p), xd, out, act_stride, out_stride, B)
    assert_close(out[:, :M], O.gemm_exact(w, x), what=f"B={B}")
    assert torch.isnan(out[:, M:]).all()             # padding untouched


@pytest.mark.parametrize("n", [4, 8])
@pytest.mark.parametrize("M,K,frac,counts", [(16, 256, 5e-2, True), (130, 512, 1e-2, False),
                                             (4096, 4096, 5e-4, False), (64, 14336, 2.5e-3, True)])
def test_batch4_batch8_escape_table(eng, O, n, M, K, frac, counts):
    """launch_split12_batch4/8_async: exact escapes from the thread-stride table; separate
    (non-strided) activation and output vectors; the per-residue counts are optional."""
    w, p, x = _case(O, M, K, 60 + n, frac=frac, B=n)
    cw = _cw(p, escape_counts=counts)
    ins = [dev(x[b].copy()) for b in range(n)]
    outs = [torch.full((M,), float("nan"), device="cuda") for _ in range(n)]
    eng.batch_matvec(cw, ins, outs)
    ref = O.gemm_exact(w, x)
    for b in range(n):
        assert_close(outs[b], ref[b], what=f"batch{n} b={b}")


def test_batch8_row_with_more_escapes_than_the_rank_list(eng, O):
    rng = np.random.default_rng(70)                              # exponents 96..135: most escape
    w = ((rng.integers(0, 2, (18, 2048)) << 15) | (rng.integers(96, 136, (18, 2048)) << 7)
         | rng.integers(0, 128, (18, 2048))).astype(np.uint16)
    p = O.pack(w)
    x = O.synth_acts(8, 2048, 70)
    assert np.diff(p.row_off).max() > 128
    ins = [dev(x[b].copy()) for b in range(8)]
    outs = [torch.empty(18, device="cuda") for _ in range(8)]
    eng.batch_matvec(_cw(p), ins, outs)
    ref = O.gemm_exact(w, x)
    for b in range(8):
        assert_close(outs[b], ref[b], what=f"b={b}")


def test_batch4_without_escapes_accepts_null_table(eng, O, golden):
    w, p = golden_packed(O, golden, "no_escapes_8x96")
    x = O.synth_acts(4, p.K, 9)
    ins = [dev(x[b].copy()) for b in range(4)]
    outs = [torch.empty(p.M, device="cuda") for _ in range(4)]
    eng.batch_matvec(_cw(p), ins, outs)               # all three table pointers are null
    ref = O.gemm_exact(w, x)
    for b in range(4):
        assert_close(outs[b], ref[b])


def test_dependent_launch_chain_gives_same_results(eng, O):
    """A chain of GEMVs whose input is the previous kernel's output buffer, with programmatic
    dependent launch on: identical to the plain launches."""
    K = M = 1024
    packs = [O.pack(O.synth_weights(M, K, 80 + i, std=0.03, outlier_frac=1e-3)) for i in range(4)]
    cws = [_cw(p) for p in packs]
    x0 = dev(O.synth_acts(1, K, 80)[0])

    def run():
        x = x0
        outs = []
        for cw in cws:
            o = torch.empty(M, device="cuda")
            eng.gemv([cw], x, [o])
            outs.append(o)
            x = o.to(torch.bfloat16).view(torch.int16)
        torch.cuda.synchronize()
        return outs

    plain = run()
    old = eng.set_dependent_launch(True)
    try:
        chained = run()
    finally:
        eng.set_dependent_launch(old)
    for a, b in zip(plain, chained):
        assert torch.equal(a, b)


def test_rejects_bad_arguments(eng, O):
    from turbo_lossless_b200 import S12Error
    w, p, x = _case(O, 16, 128, 1)
    cw, xd = _cw(p), dev(x[0])
    out = torch.empty(16, device="cuda")
    lib = eng.lib
    assert lib.nv_launch_split12_v2_async(None, cw.split_gr.data_ptr(), p.base_exp, xd.data_ptr(),
                                          out.data_ptr(), 16, 128, None) < 0
    assert lib.nv_launch_split12_v2_async(cw.split_sm.data_ptr(), cw.split_gr.data_ptr(), p.base_exp,
                                          xd.data_ptr(), out.data_ptr(), 16, 127, None) < 0
    assert b"K=127" in lib.s12_last_error()
    with pytest.raises(S12Error):
        eng.gemv_batched(cw, xd, out, 128, 16, 17)     # B outside 1..16
    assert lib.nv_launch_split12_v2_async(cw.split_sm.data_ptr(), cw.split_gr.data_ptr(), p.base_exp,
                                          xd.data_ptr(), out.data_ptr(), 0, 128, None) == 0
