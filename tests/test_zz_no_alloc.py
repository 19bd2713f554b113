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

# 8 MiB of fp32 partials / (256 sequences x 128 rows per partial tile)
MAX_CTAS_AT_B256 = (8 << 20) // (256 * 128 * 4)


def _noalloc(eng, cw, xd, M, K, B):
    got = torch.full((B, M), float("nan"), device="cuda")
    t = cw.tensor()
    rc = eng.lib.s12_gemm_noalloc_async(C.byref(t), xd.data_ptr(), K, got.data_ptr(), M, B,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, eng.lib.s12_last_error()
    torch.cuda.synchronize()
    return got


def _regular(eng, cw, xd, M, K, B):
    ref = torch.full((B, M), float("nan"), device="cuda")
    eng.gemm(cw, xd, ref, K, M, B)                    # existing entry point (cudaMalloc'd workspace)
    torch.cuda.synchronize()
    return ref


def test_noalloc_matches_regular_entry_point_twice_in_a_row(O, monkeypatch):
    from turbo_lossless_b200 import CompressedWeight, Split12Engine
    eng = Split12Engine()
    assert MAX_CTAS_AT_B256 == 64
    # First call: 14336 x 4096 at B=256 is 112 row tiles, more than the 64 CTAs whose partial tiles fit
    # the fixed array, so the launch is stream-K over 64 CTAs: 48 of them hand a partial tile to a
    # neighbour through the array.  (Fewer tiles than CTAs would run as clusters or whole tiles and
    # never touch it.)
    M, K, B = 14336, 4096, 256
    w = O.synth_weights(M, K, 11, outlier_frac=1e-3)
    cw = CompressedWeight.from_packed(O.pack(w), escape_table=False)
    x1 = O.synth_acts(B, K, 11)
    xd1 = dev(x1)
    got = _noalloc(eng, cw, xd1, M, K, B)
    assert eng.device_status() == 0
    assert_close(got, _regular(eng, cw, xd1, M, K, B).cpu().numpy(), tol=REL_TOL, what="first call")
    assert_close(got[:4], O.gemm_exact(w, x1[:4]), tol=REL_TOL, what="first call vs oracle")
    # The regular entry point, held to the same 64 CTAs and to stream-K by its tuning knobs, cuts the
    # work at the same places and therefore adds the same partials in the same order: bit-identical.
    monkeypatch.setenv("S12_GEMM_MAXGRID", str(MAX_CTAS_AT_B256))
    monkeypatch.setenv("S12_GEMM_CLUSTER", "0")
    monkeypatch.setenv("S12_GEMM_SPLIT", "0")
    same_schedule = _regular(eng, cw, xd1, M, K, B)
    monkeypatch.delenv("S12_GEMM_MAXGRID"); monkeypatch.delenv("S12_GEMM_CLUSTER"); monkeypatch.delenv("S12_GEMM_SPLIT")
    assert torch.equal(got, same_schedule)

    # Second call right after, other shape and inputs (the array still holds the first call's
    # partials): 12000 x 2048 at B=200 is 94 tiles for the 78 CTAs whose partials fit, stream-K again.
    # No device memory is allocated or freed around it.
    M2, K2, B2 = 12000, 2048, 200
    w2 = O.synth_weights(M2, K2, 12, outlier_frac=2e-3)
    cw2 = CompressedWeight.from_packed(O.pack(w2), escape_table=False)
    x2 = O.synth_acts(B2, K2, 12)
    xd2 = dev(x2)
    ref2 = _regular(eng, cw2, xd2, M2, K2, B2)
    out2 = torch.full((B2, M2), float("nan"), device="cuda")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    t2 = cw2.tensor()
    rc = eng.lib.s12_gemm_noalloc_async(C.byref(t2), xd2.data_ptr(), K2, out2.data_ptr(), M2, B2,
                                        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0, eng.lib.s12_last_error()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert eng.device_status() == 0
    assert_close(out2, ref2.cpu().numpy(), tol=REL_TOL, what="second call")
    assert_close(out2[:8], O.gemm_exact(w2, x2[:8]), tol=REL_TOL, what="second call vs oracle")
    # and the first problem once more: same bits as before
    assert torch.equal(_noalloc(eng, cw, xd1, M, K, B), got)
    assert eng.device_status() == 0


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
