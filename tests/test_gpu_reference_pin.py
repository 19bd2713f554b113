"""The CPU oracle's GEMV / GEMM statements pinned to outputs of the reference's OWN CUDA kernels.

The reference has no CPU unpack, GEMV or GEMM and no golden vectors, so the oracle functions that restate its
device arithmetic (gemm_twopass with and without the patch pass) can only be pinned by running the reference's
kernels themselves: `make -C oracle ref_gpu` compiles nvidia_kernels.cu and decompress_v2.hip unmodified for
sm_100a into oracle/_ref/libturbo_ref_gpu.so.  This file loads that library (and skips when it has not been
built), feeds it the tensors the other tests use, and checks
    reference kernel == oracle      (the pin)
    reference kernel == this library's drop-in entry point of the same name.
Only shapes on which the reference's kernels stay inside their buffers are used: M a multiple of 128, K a
multiple of 256, B equal to 32, 64 or 256 (its tile widths); its kernels read past the end of the activations and
weights for other B and M (split12_gemm_v2.cuh:125-136).  Its default dispatch is taken: the TMA kernel
(split12_gemm_v3.cuh) for B >= 64, the cp.async kernel (split12_gemm_v2.cuh) below.
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from conftest import ROOT
from gpu_util import REL_TOL, assert_close, dev

pytestmark = pytest.mark.gpu
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libturbo_ref_gpu.so")
_vp, _i = C.c_void_p, C.c_int


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libturbo_ref_gpu.so not built (make -C oracle ref_gpu next to the reference)")
    lib = C.CDLL(REF_LIB)
    lib.nv_launch_split12_v2_async.argtypes = [_vp, _vp, _i, _vp, _vp, _i, _i, _vp]
    lib.nv_launch_split12_v2_dual_async.argtypes = [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp]
    lib.nv_launch_patches_async.argtypes = [_vp] * 6 + [_i, _vp]
    lib.nv_launch_patches_batch_async.argtypes = [_vp] * 5 + [_i, _vp, _i, _vp, _i, _i, _vp]
    lib.nv_launch_split12_fused_gemm_async.argtypes = [_vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp] + [_vp] * 4
    return lib


@pytest.fixture(scope="module")
def eng():
    from turbo_lossless_b200 import Split12Engine
    return Split12Engine()


def _cw(p):
    from turbo_lossless_b200 import CompressedWeight
    return CompressedWeight.from_packed(p)


def _stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("M,K", [(4096, 4096), (1024, 4096), (256, 14336)])
def test_b1_gemv_and_patch_pass(ref, eng, O, M, K):
    w = O.synth_weights(M, K, M + K, outlier_frac=2e-3)
    p = O.pack(w)
    x = O.synth_acts(1, K, 3)
    cw, xd = _cw(p), dev(x[0])
    out = torch.full((M,), float("nan"), device="cuda")
    assert ref.nv_launch_split12_v2_async(cw.split_sm.data_ptr(), cw.split_gr.data_ptr(), p.base_exp, xd.data_ptr(),
                                          out.data_ptr(), M, K, _stream()) == 0
    torch.cuda.synchronize()
    first = out.cpu().numpy()
    assert_close(first, O.gemm_twopass(p, x, patches=False)[0], what="reference GEMV vs oracle first pass")
    assert ref.nv_launch_patches_async(cw.row_offsets.data_ptr(), cw.patch_cols.data_ptr(), cw.patch_correct.data_ptr(),
                                       cw.patch_wrong.data_ptr(), xd.data_ptr(), out.data_ptr(), M, _stream()) == 0
    torch.cuda.synchronize()
    assert_close(out, O.gemm_twopass(p, x)[0], what="reference GEMV + patches vs oracle two pass")
    assert_close(out, O.gemm_exact(w, x)[0], what="two-pass result vs exact weights")
    ours = torch.full((M,), float("nan"), device="cuda")
    eng.matvec_b1_nopatch(cw, xd, ours)
    assert_close(ours, first, what="drop-in GEMV vs reference kernel")
    eng.patches(cw, xd, ours)
    assert_close(ours, out.cpu().numpy(), what="drop-in GEMV + patches vs reference kernels")


def test_dual_gemv(ref, eng, O):
    M, K = 1024, 4096
    pa = O.pack(O.synth_weights(M, K, 31, outlier_frac=1e-3))
    pb = O.pack(O.synth_weights(M, K, 32, std=0.05))
    x = O.synth_acts(1, K, 5)
    ca, cb, xd = _cw(pa), _cw(pb), dev(x[0])
    oa, ob = torch.full((M,), float("nan"), device="cuda"), torch.full((M,), float("nan"), device="cuda")
    assert ref.nv_launch_split12_v2_dual_async(ca.split_sm.data_ptr(), ca.split_gr.data_ptr(), pa.base_exp,
                                               cb.split_sm.data_ptr(), cb.split_gr.data_ptr(), pb.base_exp,
                                               xd.data_ptr(), oa.data_ptr(), ob.data_ptr(), M, K, _stream()) == 0
    torch.cuda.synchronize()
    assert_close(oa, O.gemm_twopass(pa, x, patches=False)[0], what="reference dual a vs oracle")
    assert_close(ob, O.gemm_twopass(pb, x, patches=False)[0], what="reference dual b vs oracle")
    ua, ub = torch.empty(M, device="cuda"), torch.empty(M, device="cuda")
    eng.matvec_dual(ca, cb, xd, ua, ub)
    assert_close(ua, oa.cpu().numpy(), what="drop-in dual a vs reference kernel")
    assert_close(ub, ob.cpu().numpy(), what="drop-in dual b vs reference kernel")


@pytest.mark.parametrize("B", [32, 64, 256])
@pytest.mark.parametrize("M,K", [(4096, 4096), (1024, 4096)])
def test_fused_gemm_and_batched_patch_pass(ref, eng, O, M, K, B):
    w = O.synth_weights(M, K, M + B, outlier_frac=1e-3)
    p = O.pack(w)
    x = O.synth_acts(B, K, B)
    cw, xd = _cw(p), dev(x)
    out = torch.full((B, M), float("nan"), device="cuda")
    assert ref.nv_launch_split12_fused_gemm_async(cw.split_sm.data_ptr(), cw.split_gr.data_ptr(), p.base_exp, xd.data_ptr(), K,
                                                  out.data_ptr(), M, M, K, B, _stream(), None, None, None, None) == 0
    torch.cuda.synchronize()
    first = out.cpu().numpy()
    assert_close(first, O.gemm_twopass(p, x, patches=False), what="reference fused GEMM vs oracle first pass")
    ne = cw.patch_nonempty_rows
    assert ref.nv_launch_patches_batch_async(cw.row_offsets.data_ptr(), cw.patch_cols.data_ptr(), cw.patch_correct.data_ptr(),
                                             cw.patch_wrong.data_ptr(), ne.data_ptr(), int(ne.numel()), xd.data_ptr(), K,
                                             out.data_ptr(), M, B, _stream()) == 0
    torch.cuda.synchronize()
    assert_close(out, O.gemm_twopass(p, x), what="reference GEMM + batched patches vs oracle two pass")
    ours = torch.full((B, M), float("nan"), device="cuda")
    eng.gemm_only(cw, xd, ours, K, M, B)
    assert_close(ours, first, what="drop-in fused GEMM vs reference kernel")
    eng.patches_batch(cw, xd, ours, K, M, B)
    assert_close(ours, out.cpu().numpy(), what="drop-in GEMM + patches vs reference kernels")
    assert eng.device_status() == 0
