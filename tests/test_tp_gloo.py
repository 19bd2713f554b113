"""Tensor-parallel host logic on CPU: two gloo ranks shard a packed tensor with the library's host
helpers, each computes its share with the CPU oracle (the checker), and the exchange step is the
same all_reduce / all_gather the GPU path uses."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _shard(lib, p, kind, a, b):
    from oracle import oracle as O
    from turbo_lossless_b200.capi import S12Tensor
    t = S12Tensor()
    t.sm, t.gr = p.sm.ctypes.data, p.gr.ctypes.data
    t.row_off, t.cols = p.row_off.ctypes.data, p.cols.ctypes.data
    t.correct, t.wrong = p.correct.ctypes.data, p.wrong.ctypes.data
    t.M, t.K, t.base_exp, t.num_patches = p.M, p.K, p.base_exp, p.num_patches
    Ms, Ks = (b - a, p.K) if kind == "rows" else (p.M, b - a)
    cap = max(p.num_patches, 1)
    sm = np.zeros(Ms * Ks, np.uint8); gr = np.zeros(Ms * Ks // 2, np.uint8)
    ro = np.zeros(Ms + 1, np.int32); co = np.zeros(cap, np.int32)
    cv = np.zeros(cap, np.int16); wv = np.zeros(cap, np.int16)
    fn = lib.s12_host_shard_rows if kind == "rows" else lib.s12_host_shard_cols
    n = fn(C.byref(t), a, b, sm.ctypes.data, gr.ctypes.data, ro.ctypes.data, co.ctypes.data,
           cv.ctypes.data, wv.ctypes.data)
    assert n >= 0
    return O.Packed(Ms, Ks, p.base_exp, sm, gr, ro, co[:n].copy(), cv[:n].copy(), wv[:n].copy())


def _worker(rank, world, port, q):
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from turbo_lossless_b200 import capi
        lib = capi.load()
        M, K, B = 64, 1024, 3
        w = O.synth_weights(M, K, 5, outlier_frac=5e-3)       # same seed on every rank
        p = O.pack(w)
        x = O.synth_acts(B, K, 5)
        full = O.gemm_twopass(p, x)
        # row-parallel (o / down): column slice of the weights and of the activations, then all_reduce
        c0, c1 = rank * K // world, (rank + 1) * K // world
        part = torch.from_numpy(O.gemm_twopass(_shard(lib, p, "cols", c0, c1), x[:, c0:c1]).astype(np.float32))
        dist.all_reduce(part)
        err_row = float(np.abs(part.numpy() - full).max() / np.abs(full).max())
        # column-parallel (q/k/v, gate/up, lm_head): row slice, outputs concatenated by all_gather
        r0, r1 = rank * M // world, (rank + 1) * M // world
        mine = torch.from_numpy(np.ascontiguousarray(O.gemm_twopass(_shard(lib, p, "rows", r0, r1), x)))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        err_col = float(np.abs(torch.cat(parts, dim=1).numpy() - full).max() / np.abs(full).max())
        q.put((rank, err_row, err_col))
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_matches_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_row, err_col in res:
        assert err_row <= 1e-5, (rank, err_row)
        assert err_col <= 1e-6, (rank, err_col)


def test_bench_shard_boundaries_cover_everything():
    import bench
    for n, align in ((4096, 16), (14336, 1024), (128256, 16), (1024, 16)):
        for world in (2, 4, 8):
            spans = [bench.shard(n, r, world, align) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(lo % align == 0 for lo, _ in spans)
