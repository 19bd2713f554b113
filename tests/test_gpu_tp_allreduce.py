"""The tensor-parallel all-reduce kernel (s12_allreduce_f32_async).

On one GPU the ranks of a call run as one cooperative launch (ranks that wait on one another are
never separate launches on one device); with two or more GPUs the real path runs as one process
per GPU with the IPC handles exchanged over a gloo group.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("n", [4, 4096, 14336, 65536 + 8])
def test_emulated_ranks_one_launch(world, n):
    import torch
    from turbo_lossless_b200 import TPComm, Split12Engine
    eng = Split12Engine()
    comms = TPComm.local(world, 70000)
    rng = np.random.default_rng(world * 1000 + n)
    for call in range(3):                      # consecutive calls alternate the receive areas
        parts = [rng.standard_normal(n).astype(np.float32) for _ in range(world)]
        srcs = [torch.from_numpy(p).cuda() for p in parts]
        dsts = [torch.full((n,), float("nan"), device="cuda") for _ in range(world)]
        TPComm.all_reduce_emulated(comms, srcs, dsts)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        ref = np.zeros(n, dtype=np.float32)
        for p in parts:                        # rank order, fp32: the kernel's order of additions
            ref = ref + p
        for d in dsts:
            np.testing.assert_array_equal(d.cpu().numpy(), ref)
    for c in comms:
        c.close()


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("n", [16388, 65536 + 8, 100004])
def test_two_shot_form(monkeypatch, world, n):
    """Reduce-scatter + all-gather inside one kernel (large vectors, four ranks or more by default; forced here for
    every world): the sums are added in rank order by the part's owner, so they carry the same bits as the one-shot
    form, on every rank; consecutive calls alternate the areas; parts of a slice that do not divide evenly."""
    import torch
    from turbo_lossless_b200 import TPComm, Split12Engine
    monkeypatch.setenv("S12_COMM_TWOSHOT", "1")
    eng = Split12Engine()
    comms = TPComm.local(world, 300000)
    rng = np.random.default_rng(world * 7 + n)
    for call in range(3):
        parts = [rng.standard_normal(n).astype(np.float32) for _ in range(world)]
        srcs = [torch.from_numpy(p).cuda() for p in parts]
        dsts = [torch.full((n,), float("nan"), device="cuda") for _ in range(world)]
        TPComm.all_reduce_emulated(comms, srcs, dsts)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        ref = np.zeros(n, dtype=np.float32)
        for p in parts:
            ref = ref + p
        for d in dsts:
            np.testing.assert_array_equal(d.cpu().numpy(), ref)
    for c in comms:
        c.close()


def test_rejects_bad_sizes():
    import torch
    from turbo_lossless_b200 import TPComm, S12Error
    (c,) = TPComm.local(1, 1024)
    x = torch.zeros(2048, device="cuda")
    with pytest.raises(S12Error):
        c.all_reduce(x)                        # beyond the capacity
    with pytest.raises(S12Error):
        c.all_reduce(x[:6])                    # not a multiple of 4
    y = torch.arange(1024, device="cuda", dtype=torch.float32)
    out = c.all_reduce(y.clone())              # world of one: identity
    torch.cuda.synchronize()
    assert torch.equal(out, y)
    c.close()


@pytest.mark.parametrize("M,K", [(4096, 4096), (4096, 2048), (1000, 512), (4100, 1024)])
def test_fused_gemv_allreduce_world_of_one(M, K):
    """s12_gemv_allreduce_async on one rank: the push / signal / wait / add path of the GEMV epilogue runs
    against the rank's own receive area, and consecutive calls alternate the areas."""
    import torch
    from oracle import oracle as O
    from turbo_lossless_b200 import CompressedWeight, Split12Engine, TPComm
    eng = Split12Engine()
    (comm,) = TPComm.local(1, 8192)
    w = O.synth_weights(M, K, 5, outlier_frac=1e-3)
    cw = CompressedWeight.from_packed(O.pack(w))
    for call in range(3):
        x = O.synth_acts(1, K, 40 + call)
        xd = torch.from_numpy(x.view(np.int16)).cuda()
        out = torch.full((M,), float("nan"), device="cuda")
        comm.gemv_all_reduce(cw, xd, out)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        ref = O.gemm_exact(w, x)[0]
        np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=0, atol=1e-4 * np.abs(ref).max())
    comm.close()


@pytest.mark.parametrize("M,K,offset", [(1000, 1000, 0),      # K not a multiple of 32: the general GEMV path
                                        (1024, 1024, 4),      # activations 8 bytes off a 16-byte boundary
                                        (4096, 64, 0)])       # too small for the streaming kernel
def test_gemv_allreduce_on_shapes_the_streaming_kernel_refuses(M, K, offset):
    """Every route through s12_gemv_allreduce_async ends in the sum over ranks (here a world of one, where the
    all-reduce kernel must leave the values as they are and advance the communicator's call counter like the
    fused path does: the calls alternate between both routes and stay in step)."""
    import torch
    from oracle import oracle as O
    from turbo_lossless_b200 import CompressedWeight, Split12Engine, TPComm
    eng = Split12Engine()
    (comm,) = TPComm.local(1, 8192)
    w = O.synth_weights(M, K, 6, outlier_frac=2e-3)
    cw = CompressedWeight.from_packed(O.pack(w))
    big = O.synth_weights(4096, 4096, 7)
    cbig = CompressedWeight.from_packed(O.pack(big))
    for call in range(3):
        x = O.synth_acts(1, K, 50 + call)
        buf = torch.zeros(K + 8, dtype=torch.int16, device="cuda")
        buf[offset:offset + K] = torch.from_numpy(x[0].view(np.int16)).cuda()
        out = torch.full((M,), float("nan"), device="cuda")
        comm.gemv_all_reduce(cw, buf[offset:offset + K], out)
        xb = O.synth_acts(1, 4096, 60 + call)
        outb = torch.full((4096,), float("nan"), device="cuda")
        comm.gemv_all_reduce(cbig, torch.from_numpy(xb.view(np.int16)).cuda(), outb)   # the fused route in between
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        ref = O.gemm_exact(w, x)[0]
        np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=0, atol=1e-4 * np.abs(ref).max())
        refb = O.gemm_exact(big, xb)[0]
        np.testing.assert_allclose(outb.cpu().numpy(), refb, rtol=0, atol=1e-4 * np.abs(refb).max())
    comm.close()


@pytest.mark.parametrize("n", [4096, 65536])
def test_wait_for_a_peer_that_never_arrives_runs_out(n):
    """Rank 0 of a world of two calls the all-reduce alone with a 5 ms limit: the kernel returns, the status word
    carries 0x8000, and after both ranks reset their communicators a complete call gives the exact sum.
    (Both forms of the kernel: words with tokens for small vectors, flags for large ones.)"""
    import torch
    from turbo_lossless_b200 import TPComm, Split12Engine
    eng = Split12Engine()
    comms = TPComm.local(2, 70000)
    assert comms[0].set_wait_limit_ms(5) == 2000
    x = torch.ones(n, device="cuda")
    out = torch.empty(n, device="cuda")
    comms[0].all_reduce(x, out)                # nobody plays rank 1: nothing ever sets the awaited words
    torch.cuda.synchronize()
    assert eng.device_status() & 0x8000
    assert eng.device_status() == 0            # reading cleared it
    for c in comms:
        c.reset()
    comms[0].set_wait_limit_ms(2000)
    parts = [np.random.default_rng(r).standard_normal(n).astype(np.float32) for r in range(2)]
    srcs = [torch.from_numpy(p).cuda() for p in parts]
    dsts = [torch.full((n,), float("nan"), device="cuda") for _ in range(2)]
    TPComm.all_reduce_emulated(comms, srcs, dsts)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    for d in dsts:
        np.testing.assert_array_equal(d.cpu().numpy(), parts[0] + parts[1])
    for c in comms:
        c.close()


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("batch,vocab", [(1, 32000), (5, 1000), (64, 128256)])
def test_sharded_argmax_equals_argmax_over_the_whole_vocabulary(world, batch, vocab):
    """Output projection split by rows: local argmax with global indices, pairs collected by the all-reduce (all
    ranks emulated in one launch), merge.  Equal maxima in different shards are planted: the winner must be the one
    launch_argmax_batch picks over the unsplit logits."""
    import ctypes as C
    import torch
    from turbo_lossless_b200 import TPComm, Split12Engine
    eng = Split12Engine()
    lib = eng.lib
    rng = np.random.default_rng(world * 7 + batch)
    logits = rng.standard_normal((batch, vocab)).astype(np.float32)
    for b in range(batch):                                   # ties across (and inside) shards
        top = logits[b].max() + 1.0
        for i in rng.integers(0, vocab, 3):
            logits[b, i] = top
    full = torch.from_numpy(logits).cuda()
    want = torch.zeros(batch, dtype=torch.int32, device="cuda")
    eng.argmax(full, want)
    bounds = [(vocab // 16 * r // world) * 16 for r in range(world)] + [vocab]
    comms = TPComm.local(world, 4096 * 8)
    n = (2 * batch * world + 3) & ~3
    pairs = [torch.full((max(n, 2 * batch * world),), float("nan"), device="cuda") for _ in range(world)]
    st = torch.cuda.current_stream().cuda_stream
    shards = [full[:, bounds[r]:bounds[r + 1]].contiguous() for r in range(world)]
    for r in range(world):
        assert lib.s12_tp_argmax_partial_async(shards[r].data_ptr(), bounds[r + 1] - bounds[r], bounds[r], batch, r, world,
                                               pairs[r].data_ptr(), st) == 0
        if n > 2 * batch * world:
            pairs[r][2 * batch * world:] = 0
    TPComm.all_reduce_emulated(comms, [p[:n] for p in pairs], [p[:n] for p in pairs])
    for r in range(world):
        got = torch.full((batch,), -1, dtype=torch.int32, device="cuda")
        assert lib.s12_tp_argmax_merge_async(pairs[r].data_ptr(), world, batch, got.data_ptr(), st) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"rank {r}"
    if world == 1:                                           # the composed call on a world of one
        got = torch.full((batch,), -1, dtype=torch.int32, device="cuda")
        comms[0].tp_argmax(full, 0, got)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    assert eng.device_status() == 0
    for c in comms:
        c.close()


_WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
from turbo_lossless_b200 import TPComm, Split12Engine
eng = Split12Engine()
comm = TPComm(rank, world, 1 << 20)
ok = True
for call, n in enumerate([4096, 4096, 14336, 1 << 20, 4096, 1 << 20, 65544, 20000, 4096]):
    if call == 5:
        os.environ["S12_COMM_TWOSHOT"] = "1"                 # the reduce-scatter + all-gather form from here on
    parts = [np.random.default_rng(100 * call + r).standard_normal(n).astype(np.float32) for r in range(world)]
    x = torch.from_numpy(parts[rank]).cuda()
    out = torch.empty_like(x)
    comm.all_reduce(x, out)
    torch.cuda.synchronize()
    ref = np.zeros(n, dtype=np.float32)
    for p in parts:
        ref = ref + p
    ok = ok and np.array_equal(out.cpu().numpy(), ref) and eng.device_status() == 0
os.environ.pop("S12_COMM_TWOSHOT", None)
# row-parallel GEMV fused with its all-reduce: each rank holds a column slice of W
from oracle import oracle as O
from turbo_lossless_b200 import CompressedWeight
for call, (M, K) in enumerate([(4096, 4096), (4096, 14336), (1000, 1024), (1000, 2000)]):   # last: K/world % 32 != 0
    w = O.synth_weights(M, K, 77 + call, outlier_frac=1e-3)
    x = O.synth_acts(1, K, 5 + call)
    ks = K // world
    wr = np.ascontiguousarray(w[:, rank * ks:(rank + 1) * ks])
    cw = CompressedWeight.from_packed(O.pack(wr))
    xd = torch.from_numpy(np.ascontiguousarray(x[:, rank * ks:(rank + 1) * ks]).view(np.int16)).cuda()
    out = torch.full((M,), float("nan"), device="cuda")
    comm.gemv_all_reduce(cw, xd, out)
    torch.cuda.synchronize()
    ref = O.gemm_exact(w, x)[0]
    got = out.cpu().numpy()
    ok = ok and bool(np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()) and eng.device_status() == 0
    gathered = [None] * world
    dist.all_gather_object(gathered, got.tobytes())
    ok = ok and all(g == gathered[0] for g in gathered)      # bit-identical on every rank
# output projection split by rows: the sharded argmax equals the argmax over the gathered logits
V, Bq = 32000, 4
logits = np.random.default_rng(9).standard_normal((Bq, V)).astype(np.float32)
logits[:, 100] = logits[:, V - 7] = 50.0                     # a tie between the first and the last shard
lo, hi = V // world * rank, V // world * (rank + 1)
mine = torch.from_numpy(np.ascontiguousarray(logits[:, lo:hi])).cuda()
tok = torch.full((Bq,), -1, dtype=torch.int32, device="cuda")
comm.tp_argmax(mine, lo, tok)
want = torch.zeros(Bq, dtype=torch.int32, device="cuda")
eng.argmax(torch.from_numpy(logits).cuda(), want)
torch.cuda.synchronize()
ok = ok and torch.equal(tok, want) and eng.device_status() == 0
dist.barrier()
comm.close()
dist.destroy_process_group()
sys.exit(0 if ok else 1)
"""


def test_two_processes_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29533",
                   PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env))
    try:
        codes = [p.wait(timeout=120) for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert codes == [0, 0]
