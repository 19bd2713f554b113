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
    if M * K * B > 4096 * 4096 * 64 and B not in (64, 256):
        pytest.skip("oracle time")
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
