"""The allocation-free GEMM entry point against the regular one.

Who needs it: a host process that may not allocate device memory once it is serving -- it gave the
GPU's memory to its own pool at start-up, or it runs a latency-critical loop where cudaMalloc's locks
and implicit synchronisation are not acceptable.  `s12_gemm_noalloc_async` keeps the stream-K partial
sums in a fixed 8 MiB array inside the library instead of a cudaMalloc'd workspace.

This file is collected last on purpose: a run that stops at the first failure has then already run
every other test.  It passes on its own in a fresh process (the first call does the per-device set-up)
and after the other tests.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import REL_TOL, assert_close, dev

pytestmark = pytest.mark.gpu


def _run_pair(eng, cw, xd, M, K, B):
    ref = torch.full((B, M), float("nan"), device="cuda")
    got = torch.full((B, M), float("nan"), device="cuda")
    eng.gemm(cw, xd, ref, K, M, B)                    # existing entry point (cudaMalloc'd workspace)
    t = cw.tensor()
    rc = eng.lib.s12_gemm_noalloc_async(C.byref(t), xd.data_ptr(), K, got.data_ptr(), M, B,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, eng.lib.s12_last_error()
    torch.cuda.synchronize()
    return got, ref


def test_noalloc_matches_regular_entry_point_twice_in_a_row(O):
    from turbo_lossless_b200 import CompressedWeight, Split12Engine
    eng = Split12Engine()
    # first call: 5000 x 4096 at B=256 -- more CTAs wanted than the fixed scratch holds, so the CTA
    # count is capped at 32 and the 40 tiles are split across them (the scratch is really used)
    M, K, B = 5000, 4096, 256
    w = O.synth_weights(M, K, 11, outlier_frac=1e-3)
    cw = CompressedWeight.from_packed(O.pack(w), escape_table=False)
    x1 = O.synth_acts(B, K, 11)
    got, ref = _run_pair(eng, cw, dev(x1), M, K, B)
    assert_close(got, ref.cpu().numpy(), tol=REL_TOL, what="first call")
    assert_close(got[:8], O.gemm_exact(w, x1[:8]), tol=REL_TOL, what="first call vs oracle")
    # second call right after, other shape and inputs: the array still holds the first call's partials
    M2, K2, B2 = 1000, 2048, 48
    w2 = O.synth_weights(M2, K2, 12, outlier_frac=2e-3)
    cw2 = CompressedWeight.from_packed(O.pack(w2), escape_table=False)
    x2 = O.synth_acts(B2, K2, 12)
    got2, ref2 = _run_pair(eng, cw2, dev(x2), M2, K2, B2)
    assert_close(got2, ref2.cpu().numpy(), tol=REL_TOL, what="second call")
    assert_close(got2, O.gemm_exact(w2, x2), tol=REL_TOL, what="second call vs oracle")
    # and the first problem once more: same answer as before
    got3, _ = _run_pair(eng, cw, dev(x1), M, K, B)
    assert torch.equal(got3, got)


def test_noalloc_rejects_sizes_beyond_its_maximum(O):
    from turbo_lossless_b200 import CompressedWeight, Split12Engine
    eng = Split12Engine()
    cw = CompressedWeight.from_packed(O.pack(O.synth_weights(128, 256, 13)), escape_table=False)
    x = torch.zeros((300, 256), dtype=torch.int16, device="cuda")
    out = torch.zeros((300, 128), device="cuda")
    t = cw.tensor()
    rc = eng.lib.s12_gemm_noalloc_async(C.byref(t), x.data_ptr(), 256, out.data_ptr(), 128, 300, None)
    assert rc == -5 and b"exceeds the maximum" in eng.lib.s12_last_error()
    rc = eng.lib.s12_gemm_noalloc_async(C.byref(t), x.data_ptr(), 256, out.data_ptr(), 128, 8, None)
    assert rc == -2
