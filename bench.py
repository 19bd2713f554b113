#!/usr/bin/env python3
"""Benchmark of the split12 hot path on B200: one JSON line per run.

A "step" is one pass of the hot path over one batch of synthetic input: every
split12 projection of one decode step of the named model shape (q/k/v, o,
gate/up, down for each layer, then the output projection), fp32 outputs, called
through the library's C ABI.  Weights are random-init N(0, 0.02) bf16 generated
on the device from a seed and packed by the library's device packer (same bytes
as the reference CPU packer); they stand in for the real checkpoints.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
    python bench.py --impl reference ...      # CPU statement of the same path

Timing: blocks of exactly K steps are timed with CUDA events on the launching
stream, after W warm-up steps, and repeated until half a second of device time
has been covered; the reported time is the median block (maximum over ranks per
block).  SM clocks and throttle reasons are sampled over all blocks.

With one GPU and the default workload the line carries further blocks measured
in the same process, each with its own roofline: `b256` (Llama-3.1-8B shape at
B=256), `b16` (the default model at B=16, the small-batch range), `full_step` (every kernel of the decode step), `config1` (rotating
4096 x 4096 tensors, GEMV GB/s), `decompress` (stand-alone split12 -> bf16) and
`ref_gpu` (the reference's own CUDA kernels, when oracle/_ref holds them, timed
on the same tensors through the same entry-point names).

With N > 1 (under torchrun) the projections are tensor-parallel: q/k/v, gate/up
and the output projection are split by rows, o and down by columns, followed by
this library's all-reduce kernel over NVLink peer memory (`--comm nccl` swaps in
NCCL between graph segments).  Before timing, one step's all-reduced outputs are
compared with torch.distributed's all_reduce of the same partials (`tp_check`).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# name -> (layers, hidden, q rows, kv rows, ffn, vocab, batch)
WORKLOADS = {
    "mistral7b_b1": dict(layers=32, hidden=4096, q=4096, kv=1024, ffn=14336, vocab=32000, batch=1,
                         desc="Mistral-7B-shaped decode step at B=1 (BASELINE configs[1]): all split12 projections"),
    "mistral7b_b16": dict(layers=32, hidden=4096, q=4096, kv=1024, ffn=14336, vocab=32000, batch=16,
                          desc="Mistral-7B-shaped decode step at B=16 (the engine's small-batch range): all split12 projections"),
    "mistral7b_b32": dict(layers=32, hidden=4096, q=4096, kv=1024, ffn=14336, vocab=32000, batch=32,
                          desc="Mistral-7B-shaped decode step at B=32: all split12 projections"),
    "llama8b_b1": dict(layers=32, hidden=4096, q=4096, kv=1024, ffn=14336, vocab=128256, batch=1,
                       desc="Llama-3.1-8B-shaped decode step at B=1: all split12 projections"),
    "llama8b_b256": dict(layers=32, hidden=4096, q=4096, kv=1024, ffn=14336, vocab=128256, batch=256,
                         desc="Llama-3.1-8B-shaped decode step at B=256 (BASELINE configs[2]): all split12 projections"),
    "llama70b_b1": dict(layers=80, hidden=8192, q=8192, kv=1024, ffn=28672, vocab=128256, batch=1,
                        desc="Llama-3-70B-shaped decode step at B=1 (BASELINE configs[3]): all split12 projections"),
    "llama70b_b64": dict(layers=80, hidden=8192, q=8192, kv=1024, ffn=28672, vocab=128256, batch=64,
                         desc="Llama-3-70B-shaped decode step at B=64 (BASELINE configs[3]): all split12 projections"),
    # the whole decode step (engine/inference.cpp forward loop): the projections plus embed, norms, RoPE + INT8
    # KV store, attention at a mid-generation position, SiLU*up, argmax -- what the reference's tok/s measures
    "mistral7b_b1_full": dict(layers=32, hidden=4096, q=4096, kv=1024, ffn=14336, vocab=32000, batch=1, full=True,
                              heads=32, kv_heads=8, position=255, max_seq=384,
                              desc="Mistral-7B-shaped greedy decode step at B=1, every kernel of the step, at position 255 "
                                   "(128-token prompt + 256 generated, BASELINE configs[1])"),
    "llama8b_b256_full": dict(layers=32, hidden=4096, q=4096, kv=1024, ffn=14336, vocab=128256, batch=256, full=True,
                              heads=32, kv_heads=8, position=191, max_seq=256,
                              desc="Llama-3.1-8B-shaped greedy decode step at B=256, every kernel of the step, at position "
                                   "191 (128-token prompts + 128 generated, BASELINE configs[2])"),
    "mixtral_b64": dict(layers=32, hidden=4096, q=4096, kv=1024, ffn=14336, vocab=32000, batch=64, experts=8,
                        desc="Mixtral-8x7B-shaped decode step at B=64 (BASELINE configs[4]): attention projections, top-2 "
                             "routing over 8 packed SwiGLU experts (0.25% x100 outliers in the expert weights, uniform-random "
                             "router logits), lm_head; single GPU"),
    "config1": dict(layers=32, hidden=4096, q=4096, kv=0, ffn=0, vocab=0, batch=1,
                    desc="32 distinct 4096x4096 tensors with 0.05% x100 outliers (BASELINE configs[0] shape), one GEMV each"),
}


# (dram read + write) / packed bytes measured with ncu on one-layer runs (summaries under profiles/), per dominant kernel
TRAFFIC_RATIO = {"gemv_stream_kernel": 1.022, "gemm_tc_kernel": 1.154, "gemm_stream_kernel": 1.020}
MIN_TIMED_MS = 500.0          # blocks of K steps are repeated until this much device time is covered


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mistral7b_b1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-pdl", action="store_true", help="disable programmatic dependent launch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--blocks", default="auto", choices=["auto", "none"],
                    help="auto: the default workload also measures b256 / b16 / full_step / config1 / decompress / ref_gpu on one "
                         "GPU and a Llama-3-70B-shaped block on several; none: the named workload only")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (development only)")
    ap.add_argument("--comm", default="own", choices=["own", "fused", "nccl"],
                    help="all-reduce after the row-parallel projections at N > 1: own = this library's one-shot kernel over "
                         "peer memory as a node of the step's CUDA graph (fastest measured: the next GEMV prefetches its "
                         "weights while it runs); fused = the B=1 GEMV pushes its rows to the peers and adds them itself "
                         "(one kernel, but its CTAs stay resident while they wait); nccl = NCCL between graph segments")
    return ap.parse_args()


def peaks():
    """(HBM GB/s, sustained bf16 TFLOP/s, burst bf16 TFLOP/s, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        burst = float(p.get("bf16_tflops", 1619.0))
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops_sustained", burst)), burst, "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1400.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            time.sleep(0.25)                 # the first sample should not be later than the first timed step
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), default=None)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(sm)}


def shard(n: int, rank: int, world: int, align: int = 1):
    """[lo, hi) of rank's share of n items, boundaries multiples of `align`."""
    units = n // align
    lo = (units * rank // world) * align
    hi = (units * (rank + 1) // world) * align if rank + 1 < world else n
    return lo, hi


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2] if len(s) % 2 else 0.5 * (s[len(s) // 2 - 1] + s[len(s) // 2])


def time_blocks(torch, run, steps, warmup, world=1, dist=None, min_ms=MIN_TIMED_MS, max_blocks=40):
    """Device time of blocks of exactly `steps` calls of run(), CUDA events on the current stream, a barrier and a
    synchronize on both sides of every block.  Returns the per-block times (maximum over ranks, ms)."""
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        run()
    barrier()
    times = []
    nblocks = None
    while nblocks is None or len(times) < nblocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t[0]))
        if nblocks is None:                  # every rank derives the same count from the same (reduced) first block
            nblocks = int(min(max_blocks, max(1, -(-min_ms // max(times[0], 1e-3)))))
    return times


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------

def make_weight(torch, CompressedWeight, M, K, seed, rank=0, world=1, split=None, outlier_frac=0.0):
    """One random-init tensor generated on the device from `seed`, sharded for tensor parallelism, packed on the device."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    w = torch.randn(M, K, generator=g, device=dev) * 0.02
    if outlier_frac:
        w = torch.where(torch.rand(M, K, generator=g, device=dev) < outlier_frac, w * 100.0, w)
    w = w.to(torch.bfloat16)
    if world > 1 and split == "rows":
        lo, hi = shard(M, rank, world, 16)
        w = w[lo:hi]
    elif world > 1 and split == "cols":
        lo, hi = shard(K, rank, world, 1024 if K % (1024 * world) == 0 else 32)
        w = w[:, lo:hi]
    return CompressedWeight.pack_on_device(w.contiguous())


def build_model(cfg, rank, world, layers, torch, CompressedWeight, distinct=0):
    """Random-init weights of every projection, seeded by (layer, tensor).  distinct > 0: only that many layers are
    generated and the step cycles through them (each layer's weights are far larger than L2, so a step moves the
    same bytes from HBM; set-up of an 80-layer model is that much shorter)."""
    H, Q, KV, F, V = cfg["hidden"], cfg["q"], cfg["kv"], cfg["ffn"], cfg["vocab"]
    outlier = 5e-4 if cfg is WORKLOADS["config1"] else 0.0

    def make(M, K, seed, split, frac=outlier):
        return make_weight(torch, CompressedWeight, M, K, seed, rank, world, split, frac)

    model = {"layers": [], "lm_head": None}
    made = []
    for layer in range(layers):
        if distinct and layer >= distinct:
            model["layers"].append(made[layer % distinct])
            continue
        s = 1000 * layer
        L = {"wq": make(Q, H, s + 1, "rows")}
        if KV:
            L["wk"], L["wv"] = make(KV, H, s + 2, "rows"), make(KV, H, s + 3, "rows")
            L["wo"] = make(H, Q, s + 4, "cols")
        if F and cfg.get("experts"):
            L["experts"] = [{"w_gate": make(F, H, s + 10 * e + 15, None, 2.5e-3), "w_up": make(F, H, s + 10 * e + 16, None, 2.5e-3),
                             "w_down": make(H, F, s + 10 * e + 17, None, 2.5e-3)} for e in range(cfg["experts"])]
        elif F:
            L["w_gate"], L["w_up"] = make(F, H, s + 5, "rows"), make(F, H, s + 6, "rows")
            L["w_down"] = make(H, F, s + 7, "cols")
        model["layers"].append(L)
        made.append(L)
    if V:
        model["lm_head"] = make(V, H, 999983, "rows")
    return model


def model_tensors(model):
    out = []
    for L in model["layers"]:
        for v in L.values():
            if isinstance(v, list):                    # experts
                for ex in v:
                    out.extend(ex.values())
            else:
                out.append(v)
    if model["lm_head"] is not None:
        out.append(model["lm_head"])
    return out


def _log(msg):
    if os.environ.get("S12_BENCH_VERBOSE"):
        sys.stderr.write(f"[bench r{os.environ.get('RANK', '0')} {time.strftime('%H:%M:%S')}] {msg}\n")
        sys.stderr.flush()


class HotPath:
    """The projections of one decode step over a model built by build_model, as a replayable step."""

    def __init__(self, torch, dist, eng, model, cfg, B, rank, world, comm, comm_mode, pdl=True, graph=True):
        self.torch, self.dist, self.eng, self.model, self.B = torch, dist, eng, model, B
        self.rank, self.world, self.comm = rank, world, comm
        dev = torch.device("cuda")
        gen = torch.Generator(device=dev).manual_seed(7)
        H = cfg["hidden"]

        def act(k):
            return torch.randn(B, k, generator=gen, device=dev).to(torch.bfloat16).view(torch.int16)

        L0 = model["layers"][0]
        self.x_hidden = act(H)
        self.x_attn = act(L0["wo"].K) if "wo" in L0 else None
        self.x_ffn = act(L0["w_down"].K) if "w_down" in L0 else None
        self.o_q = torch.empty(B, L0["wq"].M, device=dev)
        self.o_k = torch.empty(B, L0["wk"].M, device=dev) if "wk" in L0 else None
        self.o_v = torch.empty(B, L0["wv"].M, device=dev) if "wv" in L0 else None
        self.o_o = torch.empty(B, H, device=dev)
        self.o_g = torch.empty(B, L0["w_gate"].M, device=dev) if "w_gate" in L0 else None
        self.o_u = torch.empty(B, L0["w_up"].M, device=dev) if "w_up" in L0 else None
        self.o_d = torch.empty(B, H, device=dev)
        self.logits = torch.empty(B, model["lm_head"].M, device=dev) if model["lm_head"] is not None else self.o_q
        self.tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.launches = 0
        self.sharded_argmax = False
        self.vocab_lo = shard(cfg["vocab"], rank, world, 16)[0] if cfg["vocab"] else 0
        self.use_fused = comm is not None and comm_mode == "fused" and B == 1
        self.moe_blocks, self.router_logits = [], None
        if cfg.get("experts"):
            from turbo_lossless_b200.moe import MoEFeedForward
            self.router_logits = torch.rand(B, cfg["experts"], generator=gen, device=dev)
            self.moe_blocks = [MoEFeedForward(L["experts"], B, eng=eng) for L in model["layers"]]
        self.segments = []
        self._build()
        self.pdl, self.want_graph = pdl, graph
        self.graph = None

    # -- the step as a list of segments: ("k", fn) = our launches only (capturable as one CUDA graph), ("ar", tensor)
    # = an NCCL all-reduce after a row-parallel projection.  With --comm own (default) the all-reduce is a kernel of
    # this library and the whole step stays one graph.  NCCL collectives are kept out of graph capture (capturing
    # them hung on this pool), so with --comm nccl a step replays one small graph per segment.
    def _proj(self, ws, x, outs):
        if self.B == 1:
            self.eng.gemv(ws, x, outs)
        else:
            self.eng.gemm_multi(ws, x, outs, x.shape[1], self.B)
        self.launches += 1

    def _add_k(self, fn):
        if self.segments and self.segments[-1][0] == "k":
            prev = self.segments[-1][1]
            self.segments[-1] = ("k", lambda prev=prev, fn=fn: (prev(), fn()))
        else:
            self.segments.append(("k", fn))

    def _all_reduce(self, t):
        if self.comm is not None:
            def ar(t=t):
                self.comm.all_reduce(t)
                self.launches += 1
            self._add_k(ar)
        else:
            self.segments.append(("ar", t))

    def _fused(self, w, x, out):
        self.comm.gemv_all_reduce(w, x, out)
        self.launches += 1

    def _moe_layer(self, L, blk):
        self._proj([L["wq"], L["wk"], L["wv"]], self.x_hidden, [self.o_q, self.o_k, self.o_v])
        self._proj([L["wo"]], self.x_attn, [self.o_o])
        blk.forward(self.x_hidden, self.router_logits, self.o_d)
        self.launches += blk.launches

    def _build(self):
        m, world = self.model, self.world
        for L, blk in zip(m["layers"], self.moe_blocks):
            self._add_k(lambda L=L, blk=blk: self._moe_layer(L, blk))
        for L in ([] if self.moe_blocks else m["layers"]):
            if "wk" in L:
                self._add_k(lambda L=L: self._proj([L["wq"], L["wk"], L["wv"]], self.x_hidden, [self.o_q, self.o_k, self.o_v]))
                if self.use_fused:
                    self._add_k(lambda L=L: self._fused(L["wo"], self.x_attn, self.o_o))
                else:
                    self._add_k(lambda L=L: self._proj([L["wo"]], self.x_attn, [self.o_o]))
                    if world > 1:
                        self._all_reduce(self.o_o)
            else:
                self._add_k(lambda L=L: self._proj([L["wq"]], self.x_hidden, [self.o_q]))
            if "w_gate" in L:
                self._add_k(lambda L=L: self._proj([L["w_gate"], L["w_up"]], self.x_hidden, [self.o_g, self.o_u]))
                if self.use_fused:
                    self._add_k(lambda L=L: self._fused(L["w_down"], self.x_ffn, self.o_d))
                else:
                    self._add_k(lambda L=L: self._proj([L["w_down"]], self.x_ffn, [self.o_d]))
                    if world > 1:
                        self._all_reduce(self.o_d)
        if m["lm_head"] is not None:
            self._add_k(lambda: self._proj([m["lm_head"]], self.x_hidden, [self.logits]))
            if world > 1 and self.comm is not None:
                # the output projection is split by rows: local argmax + the ranks' best pairs through the all-reduce
                def tp_argmax():
                    self.comm.tp_argmax(self.logits, self.vocab_lo, self.tokens)
                    self.launches += 3
                self._add_k(tp_argmax)
                self.sharded_argmax = True

    def step(self):
        for kind, item in self.segments:
            if kind == "k":
                item()
            else:
                self.dist.all_reduce(item)

    def prepare(self, stream):
        """First eager step (loads every kernel), then capture.  Returns the callable that runs one step."""
        torch = self.torch
        self.eng.set_dependent_launch(self.pdl)
        self.launches = 0
        self.step()
        torch.cuda.synchronize()
        self.launches_per_step = self.launches
        if self.want_graph:
            try:
                graphs = []
                for kind, item in self.segments:
                    if kind != "k":
                        graphs.append((kind, item))
                        continue
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        item()
                    graphs.append(("g", g))
                self.graph = graphs
            except Exception as e:               # eager launches still measure the same work
                sys.stderr.write(f"[bench] graph capture failed ({e}); launching eagerly\n")
                self.graph = None
                torch.cuda.synchronize()
        if self.graph is None:
            return self.step

        def replay():
            for kind, item in self.graph:
                if kind == "g":
                    item.replay()
                else:
                    self.dist.all_reduce(item)
        return replay

    def argmax(self):
        """Greedy token of every sequence from the logits (the engine's launch_argmax_batch)."""
        self.eng.argmax(self.logits, self.tokens)


def roofline_hbm(gbs, hbm_peak, src, kernel, alg_bytes, traffic_ratio=None):
    r = {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(gbs / hbm_peak, 4),
         "traffic": int(alg_bytes * traffic_ratio) if traffic_ratio else None, "peak_source": src, "kernel": kernel,
         "algorithmic_bytes": int(alg_bytes), "frac_of_nominal_8TBps": round(gbs / 8000.0, 4)}
    if traffic_ratio:
        r["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum on a one-layer run, scaled by packed bytes"
    return r


def roofline_tensor(tflops, sustained, burst, src, kernel, alg_bytes, traffic_ratio=None):
    r = {"bound": "tensor", "achieved": round(tflops, 2), "peak": sustained, "unit": "TFLOP/s", "frac": round(tflops / sustained, 4),
         "frac_of_burst_peak": round(tflops / burst, 4), "burst_peak": burst,
         "traffic": int(alg_bytes * traffic_ratio) if traffic_ratio else None, "peak_source": src + ", sustained figure",
         "kernel": kernel, "algorithmic_bytes": int(alg_bytes)}
    if traffic_ratio:
        r["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum on a one-layer run, scaled by packed bytes"
    return r


def measure_hot_path(torch, dist, hp, stream, steps, warmup, world, e2e_argmax):
    """Timed blocks of the hot path, then the end-to-end loop (pinned host activations in, result back, every step)."""
    run = hp.prepare(stream)
    times = time_blocks(torch, run, steps, warmup, world, dist)
    B = hp.B
    x_host = torch.empty(hp.x_hidden.shape, dtype=torch.int16).pin_memory()
    x_host.copy_(hp.x_hidden.cpu())
    if e2e_argmax:
        res_host = torch.zeros(B, dtype=torch.int32).pin_memory()
        res_dev = hp.tokens
    else:
        res_host = torch.empty(hp.logits.shape, dtype=torch.float32).pin_memory()
        res_dev = hp.logits

    def enqueue():
        hp.x_hidden.copy_(x_host, non_blocking=True)
        hp.step()
        if e2e_argmax and not hp.sharded_argmax:
            hp.argmax()
        res_host.copy_(res_dev, non_blocking=True)

    # the user-facing call of a decode loop: copy the step's input in, run the step, take the token on the device,
    # copy it out -- captured as one CUDA graph when the whole step is capturable (no NCCL segment in it)
    e2e_graph = None
    if hp.graph is not None and all(kind == "g" for kind, _ in hp.graph):
        try:
            launches_before = hp.launches
            e2e_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(e2e_graph, stream=stream):
                enqueue()
            hp.launches = launches_before
        except Exception as e:
            sys.stderr.write(f"[bench] end-to-end graph capture failed ({e}); launching its parts one by one\n")
            e2e_graph = None
            torch.cuda.synchronize()

    def e2e_step():
        if e2e_graph is not None:
            e2e_graph.replay()
        else:
            hp.x_hidden.copy_(x_host, non_blocking=True)
            run()
            if e2e_argmax and not hp.sharded_argmax:
                hp.argmax()
            res_host.copy_(res_dev, non_blocking=True)
        stream.synchronize()

    for _ in range(2):
        e2e_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    if world > 1:
        dist.barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e = {"value": round(B * steps / float(t[0]) * 1e3, 2), "unit": "tok/s",
           "h2d_bytes_per_step": int(x_host.numel() * 2), "d2h_bytes_per_step": int(res_host.numel() * res_host.element_size()),
           "result": "greedy token ids (device argmax over the logits)" if e2e_argmax else "fp32 logits",
           "launch": "one CUDA graph: H2D copy, step, argmax, D2H copy" if e2e_graph is not None else "copies and launches issued one by one"}
    return times, e2e


def tp_check(torch, dist, eng, comm, model, hp, rank, world):
    """One layer's row-parallel outputs and the sharded output projection, before timing: this library's all-reduce
    against torch.distributed's all_reduce of the same partial results, and bit-identity of the sums across ranks."""
    worst, identical = 0.0, True
    L = model["layers"][0]
    for name, x, out in (("wo", hp.x_attn, hp.o_o), ("w_down", hp.x_ffn, hp.o_d)):
        if name not in L:
            continue
        if hp.B == 1:
            eng.gemv([L[name]], x, [out])
        else:
            eng.gemm_multi([L[name]], x, [out], x.shape[1], hp.B)
        torch.cuda.synchronize()
        ref = out.clone()
        dist.all_reduce(ref)
        mine = out.clone()
        if comm is not None:
            comm.all_reduce(mine)
        else:
            dist.all_reduce(mine)
        torch.cuda.synchronize()
        scale = float(ref.abs().max()) or 1.0
        worst = max(worst, float((mine - ref).abs().max()) / scale)
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        identical = identical and all(torch.equal(g, gathered[0]) for g in gathered)
    argmax_ok = None
    if comm is not None and model["lm_head"] is not None:
        if hp.B == 1:
            eng.gemv([model["lm_head"]], hp.x_hidden, [hp.logits])
        else:
            eng.gemm_multi([model["lm_head"]], hp.x_hidden, [hp.logits], hp.x_hidden.shape[1], hp.B)
        comm.tp_argmax(hp.logits, hp.vocab_lo, hp.tokens)
        torch.cuda.synchronize()
        sizes = torch.tensor([hp.logits.shape[1]], device="cuda")
        all_sizes = [torch.zeros_like(sizes) for _ in range(world)]
        dist.all_gather(all_sizes, sizes)
        widest = int(max(int(x[0]) for x in all_sizes))
        padded = torch.full((hp.B, widest), float("-inf"), device="cuda")
        padded[:, :hp.logits.shape[1]] = hp.logits
        gathered = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(gathered, padded)
        whole = torch.cat([g[:, :int(n[0])] for g, n in zip(gathered, all_sizes)], dim=1)
        argmax_ok = bool(torch.equal(whole.argmax(dim=1).to(torch.int32), hp.tokens))
    t = torch.tensor([worst, 0.0 if identical else 1.0, 0.0 if argmax_ok in (None, True) else 1.0], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {"max_rel_err": float(t[0]), "bit_identical_across_ranks": float(t[1]) == 0.0, "tolerance": 1e-5,
           "ok": float(t[0]) <= 1e-5 and float(t[1]) == 0.0 and float(t[2]) == 0.0,
           "what": "layer 0 o and down projections: own all-reduce vs torch.distributed all_reduce of the same partials"}
    if argmax_ok is not None:
        out["sharded_argmax_equals_argmax_of_gathered_logits"] = float(t[2]) == 0.0
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from turbo_lossless_b200 import CompressedWeight, Split12Engine, TPComm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = WORKLOADS[args.workload]
    if cfg.get("experts") and world > 1:
        raise SystemExit("mixtral_b64 runs on one GPU (expert weights are not sharded)")
    layers = args.layers or cfg["layers"]
    B, H = cfg["batch"], cfg["hidden"]
    eng = Split12Engine()
    eng.init()
    comm_floats = max(B * H, 256 * 8192)
    comm = TPComm(rank, world, comm_floats) if (world > 1 and args.comm != "nccl") else None
    _log("process group up; building model")
    model = build_model(cfg, rank, world, layers, torch, CompressedWeight)
    _log("model packed")
    tensors = model_tensors(model)
    comp_bytes = sum(t.compressed_bytes for t in tensors)             # this rank
    weights = sum(t.M * t.K for t in tensors)
    torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    hbm_peak, tf_sus, tf_burst, peak_src = peaks()
    extra = {}
    with torch.cuda.stream(stream):
        hp = HotPath(torch, dist, eng, model, cfg, B, rank, world, comm, args.comm, pdl=not args.no_pdl, graph=not args.no_graph)
        check = tp_check(torch, dist, eng, comm, model, hp, rank, world) if world > 1 else None
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        # the step's result is the greedy token, taken on the device as the engine does (launch_argmax, engine/inference.cpp)
        times, e2e = measure_hot_path(torch, dist, hp, stream, args.steps, args.warmup, world,
                                      e2e_argmax=bool(cfg["vocab"]) or hp.sharded_argmax)
        clocks = sampler.stop() if rank == 0 else None
        ms = median(times)
        _log(f"timed region done: {ms / args.steps:.3f} ms/step over {len(times)} blocks")

        tot = torch.tensor([float(comp_bytes), float(weights)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        total_bytes, total_weights = float(tot[0]), float(tot[1])

        # the same step without programmatic dependent launch: launches then run strictly one after the other, as they
        # do under a profiler, so this is the figure that per-launch profiler times add up to
        no_pdl = None
        if world == 1 and not args.no_pdl and not args.no_graph:
            hp2 = HotPath(torch, dist, eng, model, cfg, B, rank, world, comm, args.comm, pdl=False, graph=True)
            run2 = hp2.prepare(stream)
            t2 = median(time_blocks(torch, run2, args.steps, 2, min_ms=100.0)) / args.steps
            no_pdl = {"ms_per_step": round(t2, 4), "launches_per_step": hp2.launches_per_step,
                      "us_per_launch": round(1e3 * t2 / hp2.launches_per_step, 2)}
            del hp2, run2
            eng.set_dependent_launch(not args.no_pdl)

        if args.blocks == "auto" and args.workload == "mistral7b_b1" and not args.layers:
            if world == 1:
                extra = single_gpu_blocks(torch, eng, model, args, stream, CompressedWeight)
            else:
                extra = {"llama70b_b1": tp_70b_block(torch, dist, eng, comm, args, stream, rank, world, CompressedWeight, TPComm)}
    status = eng.device_status()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_step = ms / args.steps
    toks = B * 1e3 / ms_step
    per_gpu_gbs = (total_bytes / world) / (ms_step * 1e-3) / 1e9
    kernel = "gemv_stream_kernel" if B == 1 else ("gemm_tc_kernel" if B > 16 else "gemm_stream_kernel")
    if B >= 128:
        roof = roofline_tensor(2.0 * total_weights * B / world / (ms_step * 1e-3) / 1e12, tf_sus, tf_burst, peak_src, kernel,
                               total_bytes / world, TRAFFIC_RATIO.get(kernel))
    else:
        roof = roofline_hbm(per_gpu_gbs, hbm_peak, peak_src, kernel, total_bytes / world, TRAFFIC_RATIO.get(kernel))

    line = {
        "metric": "tok/s", "value": round(toks, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 weights (split12), fp32 accumulate",
        "data": "synthetic: seeded N(0,0.02) bf16 weights packed to split12 on the device; random bf16 activations",
        "config": {"workload": args.workload, "what": cfg["desc"], "layers": layers, "batch": B,
                   "parallelism": f"tp{world}" if world > 1 else "single",
                   "collective": ("none" if world == 1 else
                                  ("row-parallel GEMV fused with its one-shot all-reduce over NVLink peer memory (one kernel)" if hp.use_fused
                                   else "one-shot all-reduce kernel over NVLink peer memory, inside the step's graph") if comm is not None
                                  else "NCCL all_reduce between graph segments"),
                   "l2": "inputs larger than L2 (packed weights of one step: %.2f GB per GPU)" % (total_bytes / world / 1e9),
                   "launch": ("cuda graph" if hp.graph is not None else "eager") + ("" if args.no_pdl else " + programmatic dependent launch"),
                   "timing": f"median of {len(times)} blocks of {args.steps} steps each (CUDA events, max over ranks per block)",
                   "excluded": "norm/rope/attention/argmax kernels between the projections are not timed here (full_step times the whole step)"},
        "timing_blocks_ms": {"n": len(times), "min": round(min(times), 3), "median": round(ms, 3), "max": round(max(times), 3)},
        "compressed_GBps_per_gpu": round(per_gpu_gbs, 1),
        "roofline": roof,
        "e2e": e2e,
        "gpu_launches": hp.launches_per_step * args.steps * len(times),
        "clocks": clocks, "device_status": status,
    }
    if no_pdl:
        line["no_dependent_launch"] = no_pdl
    if check is not None:
        line["tp_check"] = check
    line.update(extra)
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, layers, B, seconds=12.0)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# further blocks of the default run
# ----------------------------------------------------------------------------------------------

def single_gpu_blocks(torch, eng, model, args, stream, CompressedWeight):
    hbm_peak, tf_sus, tf_burst, peak_src = peaks()
    out = {}
    steps = args.steps

    # ---- b256: Llama-3.1-8B shape at B = 256 (the layers have Mistral-7B's shapes; the output projection is 128256 rows)
    cfg = WORKLOADS["llama8b_b256"]
    lm = make_weight(torch, CompressedWeight, cfg["vocab"], cfg["hidden"], 999984)
    m2 = {"layers": model["layers"], "lm_head": lm}
    hp = HotPath(torch, None, eng, m2, cfg, cfg["batch"], 0, 1, None, "own")
    sampler = ClockSampler(torch.cuda.current_device()); sampler.start()
    times, e2e = measure_hot_path(torch, None, hp, stream, steps, max(args.warmup, 3), 1, e2e_argmax=True)
    clocks = sampler.stop()
    ms_step = median(times) / steps
    tens = model_tensors(m2)
    w = float(sum(t.M * t.K for t in tens)); by = float(sum(t.compressed_bytes for t in tens))
    tf = 2.0 * w * cfg["batch"] / (ms_step * 1e-3) / 1e12
    out["b256"] = {"workload": "llama8b_b256", "what": cfg["desc"], "value": round(cfg["batch"] * 1e3 / ms_step, 1), "unit": "tok/s",
                   "ms_per_step": round(ms_step, 4), "tflops": round(tf, 1),
                   "roofline": roofline_tensor(tf, tf_sus, tf_burst, peak_src, "gemm_tc_kernel", by, TRAFFIC_RATIO["gemm_tc_kernel"]),
                   "e2e": e2e, "gpu_launches": hp.launches_per_step * steps * len(times), "clocks": clocks,
                   "timing_blocks_ms": {"n": len(times), "min": round(min(times), 3), "max": round(max(times), 3)}}
    del hp, m2, lm
    torch.cuda.empty_cache()

    # ---- b16: the same model at B = 16, the small-batch range (HBM-bound: streaming kernel on the tensors of 48 row
    # tiles or more, the GEMV family on the 4096-row ones)
    cfg = WORKLOADS["mistral7b_b16"]
    hp = HotPath(torch, None, eng, model, cfg, cfg["batch"], 0, 1, None, "own")
    times, e2e = measure_hot_path(torch, None, hp, stream, steps, max(args.warmup, 3), 1, e2e_argmax=True)
    ms_step = median(times) / steps
    tens = model_tensors(model)
    by = float(sum(t.compressed_bytes for t in tens))
    out["b16"] = {"workload": "mistral7b_b16", "what": cfg["desc"], "value": round(cfg["batch"] * 1e3 / ms_step, 1), "unit": "tok/s",
                  "ms_per_step": round(ms_step, 4),
                  "roofline": roofline_hbm(by / (ms_step * 1e-3) / 1e9, hbm_peak, peak_src, "gemm_stream_kernel", by,
                                           TRAFFIC_RATIO.get("gemm_stream_kernel")),
                  "e2e": e2e, "gpu_launches": hp.launches_per_step * steps * len(times),
                  "timing_blocks_ms": {"n": len(times), "min": round(min(times), 3), "max": round(max(times), 3)}}
    del hp
    torch.cuda.empty_cache()

    # ---- full_step: every kernel of the Mistral-7B-shaped decode step at B = 1
    out["full_step"] = full_step_block(torch, eng, model, WORKLOADS["mistral7b_b1_full"], steps, max(args.warmup, 3), stream)

    # ---- config1: 4096 x 4096 tensors with 0.05 % x100 outliers, one GEMV each
    K = M = 4096
    tensors = [make_weight(torch, CompressedWeight, M, K, 5000 + i, outlier_frac=5e-4) for i in range(32)]
    x = torch.randn(1, K, device="cuda").to(torch.bfloat16).view(torch.int16)
    y = torch.empty(M, device="cuda")
    by = float(M * K * 1.5)
    res = {}
    for name, seq in (("rotating", tensors), ("l2_resident", [tensors[0]] * 32)):
        def step(seq=seq):
            for t in seq:
                eng.gemv([t], x[0], [y])
        step(); torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            step()
        ms = median(time_blocks(torch, g.replay, steps, 3, min_ms=200.0)) / steps
        res[name] = by * 32 / (ms * 1e-3) / 1e9
    esc = sum(t.num_patches for t in tensors) / (32.0 * M * K)
    out["config1"] = {"what": WORKLOADS["config1"]["desc"] + "; 32 tensors = 805 MB rotate so that reads miss L2",
                      "value": round(res["rotating"], 1), "unit": "GB/s", "escape_rate": round(esc, 6),
                      "us_per_gemv": round(by / res["rotating"] / 1e3, 2),
                      "l2_resident_GBps": round(res["l2_resident"], 1),
                      "l2_resident_note": "the same 25 MB tensor 32 times: served by L2, not an HBM figure",
                      "roofline": roofline_hbm(res["rotating"], hbm_peak, peak_src, "gemv_stream_kernel", by * 32, TRAFFIC_RATIO["gemv_stream_kernel"]),
                      "gpu_launches": 32 * steps}
    del tensors

    # ---- decompress: stand-alone lossless split12 -> bf16 (replaces nv_decode_split12_to_bf16, nvidia_kernels.cu:533-548)
    ws = [L[n] for L in model["layers"][:4] for n in ("w_gate", "w_up")]            # 8 tensors of 14336 x 4096: 0.7 GB packed
    outs = [torch.empty(t.M * t.K, dtype=torch.int16, device="cuda") for t in ws]   # 0.94 GB of bf16
    def dstep():
        for t, o in zip(ws, outs):
            eng.decompress(t, o)
    dstep(); torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        dstep()
    ms = median(time_blocks(torch, g.replay, max(2, steps // 4), 3, min_ms=200.0)) / max(2, steps // 4)
    n = float(sum(t.M * t.K for t in ws))
    gbs = 3.5 * n / (ms * 1e-3) / 1e9
    out["decompress"] = {"what": "s12_decompress_async over 8 gate/up tensors (14336 x 4096, escapes patched in the same kernel), "
                                 "1.5 B read + 2 B written per weight; 0.7 GB in, 0.94 GB out per pass: larger than L2",
                         "value": round(gbs, 1), "unit": "GB/s", "weights_per_s": round(n / (ms * 1e-3) / 1e9, 1),
                         "weights_per_s_unit": "G weights/s",
                         "roofline": roofline_hbm(gbs, hbm_peak, peak_src, "decompress16_kernel", 3.5 * n), "gpu_launches": len(ws) * max(2, steps // 4)}
    del outs
    torch.cuda.empty_cache()

    out["ref_gpu"] = ref_gpu_block(torch, eng, model, stream)
    return out


def full_step_block(torch, eng, model, cfg, steps, warmup, stream):
    from turbo_lossless_b200 import Decoder, DecoderConfig
    hbm_peak, tf_sus, tf_burst, peak_src = peaks()
    layers, B, H, V = len(model["layers"]), cfg["batch"], cfg["hidden"], cfg["vocab"]
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(11)
    dc = DecoderConfig(n_embd=H, n_head=cfg["heads"], n_head_kv=cfg["kv_heads"], n_ff=cfg["ffn"], n_vocab=V, n_layer=layers,
                       max_seq=cfg["max_seq"])
    embd = torch.randn(V, H, generator=gen, device=dev).to(torch.bfloat16).view(torch.int16)
    names = [f"attn_norm.{i}" for i in range(layers)] + [f"ffn_norm.{i}" for i in range(layers)] + ["output_norm"]
    norms = {nm: 1.0 + 0.1 * torch.randn(H, generator=gen, device=dev) for nm in names}
    dec = Decoder(dc, model["layers"], model["lm_head"], embd, norms, batch=B, eng=eng)
    pos = cfg["position"]
    dec.kv_k.copy_(torch.randint(-127, 128, dec.kv_k.shape, generator=gen, device=dev, dtype=torch.int8))
    dec.kv_v.copy_(torch.randint(-127, 128, dec.kv_v.shape, generator=gen, device=dev, dtype=torch.int8))
    dec.sc_k.fill_(0.02); dec.sc_v.fill_(0.02)
    dec.positions.fill_(pos)
    tok_host = torch.randint(0, V, (B,), dtype=torch.int32).pin_memory()
    out_host = torch.zeros(B, dtype=torch.int32).pin_memory()
    dec.tokens.copy_(tok_host)
    dec.forward(attn_len=pos + 1)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        dec.forward(attn_len=pos + 1)
    times = time_blocks(torch, graph.replay, steps, warmup)
    ms_step = median(times) / steps

    def e2e_step():
        dec.tokens.copy_(tok_host, non_blocking=True)
        graph.replay()
        out_host.copy_(dec.next_tokens, non_blocking=True)
        stream.synchronize()
    for _ in range(2):
        e2e_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    tens = model_tensors(model)
    by = float(sum(t.compressed_bytes for t in tens))
    gbs = by / (ms_step * 1e-3) / 1e9
    roof = roofline_hbm(gbs, hbm_peak, peak_src, "gemv_stream_kernel", by, TRAFFIC_RATIO["gemv_stream_kernel"])
    roof["note"] = "projection bytes over the time of the WHOLE step (attention, norms, RoPE, argmax included in the time only)"
    return {"workload": "mistral7b_b1_full", "what": cfg["desc"], "value": round(B * 1e3 / ms_step, 2), "unit": "tok/s",
            "ms_per_step": round(ms_step, 4), "roofline": roof,
            "e2e": {"value": round(B * steps / e2e_s, 2), "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                    "result": "greedy token ids"},
            "gpu_launches": dec.launches_per_step() * steps * len(times)}


def ref_gpu_block(torch, eng, model, stream):
    """The reference's own CUDA kernels (nvidia_kernels.cu compiled unmodified for sm_100a into oracle/_ref) next to this
    library's, on the same packed tensors, through the entry points of the same names, launched eagerly and timed with
    CUDA events over 8 rotating 14336 x 4096 tensors (0.7 GB: reads miss L2).  A baseline leg, not the product path."""
    path = os.path.join(ROOT, "oracle", "_ref", "libturbo_ref_gpu.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libturbo_ref_gpu.so is not built (needs the reference checkout at build time)"}
    ref = C.CDLL(path)
    vp, ci = C.c_void_p, C.c_int
    gemv_sig = [vp, vp, ci, vp, vp, ci, ci, vp]
    gemm_sig = [vp, vp, ci, vp, ci, vp, ci, ci, ci, ci, vp] + [vp] * 4
    ws = [L[n] for L in model["layers"][:4] for n in ("w_gate", "w_up")]
    M, K, B = ws[0].M, ws[0].K, 256
    x1 = torch.randn(1, K, device="cuda").to(torch.bfloat16).view(torch.int16)
    xb = torch.randn(B, K, device="cuda").to(torch.bfloat16).view(torch.int16)
    y1 = torch.empty(M, device="cuda")
    yb = torch.empty(B, M, device="cuda")
    st = stream.cuda_stream
    res = {}
    old = eng.set_dependent_launch(False)
    for who, lib in (("reference", ref), ("ours", eng.lib)):
        lib.nv_launch_split12_v2_async.argtypes = gemv_sig
        lib.nv_launch_split12_fused_gemm_async.argtypes = gemm_sig

        def gemv(lib=lib):
            for t in ws:
                lib.nv_launch_split12_v2_async(t.split_sm.data_ptr(), t.split_gr.data_ptr(), t.base_exp, x1.data_ptr(), y1.data_ptr(), M, K, st)

        def gemm(lib=lib):
            for t in ws:
                lib.nv_launch_split12_fused_gemm_async(t.split_sm.data_ptr(), t.split_gr.data_ptr(), t.base_exp, xb.data_ptr(), K,
                                                       yb.data_ptr(), M, M, K, B, st, None, None, None, None)
        for name, fn in (("gemv", gemv), ("gemm", gemm)):
            ms = median(time_blocks(torch, fn, 3, 2, min_ms=60.0)) / 3 / len(ws)
            res[(who, name)] = ms * 1e3
    eng.set_dependent_launch(old)
    by, fl = 1.5 * M * K, 2.0 * M * K * B
    return {"what": f"{M} x {K} tensor, escapes left 'wrong' (the engine's first pass); GEMV at B=1, fused GEMM at B={B}; eager launches",
            "gemv": {"reference_us": round(res[("reference", "gemv")], 1), "ours_us": round(res[("ours", "gemv")], 1),
                     "reference_GBps": round(by / res[("reference", "gemv")] / 1e3, 1), "ours_GBps": round(by / res[("ours", "gemv")] / 1e3, 1),
                     "reference_kernel": "nv_split12_matvec_multirow (nvidia_kernels.cu:102-175)"},
            "gemm": {"reference_us": round(res[("reference", "gemm")], 1), "ours_us": round(res[("ours", "gemm")], 1),
                     "reference_tflops": round(fl / res[("reference", "gemm")] / 1e6, 1), "ours_tflops": round(fl / res[("ours", "gemm")] / 1e6, 1),
                     "reference_kernel": "split12_fused_gemm_v3 (split12_gemm_v3.cuh:111-253)"}}


def tp_70b_block(torch, dist, eng, comm, args, stream, rank, world, CompressedWeight, TPComm):
    """BASELINE configs[3] at B = 1 on the ranks of this run: 80 layers of the Llama-3-70B shapes, of which 8 are
    generated and the step cycles through them (the same bytes leave HBM; one layer's shard is far larger than L2)."""
    cfg = WORKLOADS["llama70b_b1"]
    hbm_peak, tf_sus, tf_burst, peak_src = peaks()
    model = build_model(cfg, rank, world, cfg["layers"], torch, CompressedWeight, distinct=8)
    hp = HotPath(torch, dist, eng, model, cfg, 1, rank, world, comm, args.comm)
    check = tp_check(torch, dist, eng, comm, model, hp, rank, world)
    steps = max(4, args.steps // 2)
    times, e2e = measure_hot_path(torch, dist, hp, stream, steps, 3, world, e2e_argmax=hp.sharded_argmax)
    ms_step = median(times) / steps
    tens = model_tensors(model)
    tot = torch.tensor([float(sum(t.compressed_bytes for t in tens))], device="cuda", dtype=torch.float64)
    dist.all_reduce(tot)
    by = float(tot[0]) / world
    gbs = by / (ms_step * 1e-3) / 1e9
    return {"workload": "llama70b_b1", "what": cfg["desc"] + "; 8 distinct layers cycled 10 times", "value": round(1e3 / ms_step, 2),
            "unit": "tok/s", "ms_per_step": round(ms_step, 4), "n_gpus": world,
            "roofline": roofline_hbm(gbs, hbm_peak, peak_src, "gemv_stream_kernel", by, TRAFFIC_RATIO["gemv_stream_kernel"]),
            "e2e": e2e, "tp_check": check, "gpu_launches": hp.launches_per_step * steps * len(times)}


def run_full(args):
    """Whole decode step through turbo_lossless_b200.decoder.Decoder, one GPU."""
    import torch
    from turbo_lossless_b200 import CompressedWeight, Split12Engine
    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"unavailable": "the *_full workloads run on one GPU"}), flush=True)
        return
    torch.cuda.set_device(0)
    cfg = WORKLOADS[args.workload]
    layers = args.layers or cfg["layers"]
    B = cfg["batch"]
    eng = Split12Engine()
    eng.init()
    model = build_model(cfg, 0, 1, layers, torch, CompressedWeight)
    eng.set_dependent_launch(not args.no_pdl)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        sampler = ClockSampler(0)
        sampler.start()
        blk = full_step_block(torch, eng, model, cfg, args.steps, args.warmup, stream)
        clocks = sampler.stop()
    status = eng.device_status()
    roof = blk["roofline"]
    if B >= 128:
        hbm_peak, tf_sus, tf_burst, peak_src = peaks()
        w = float(sum(t.M * t.K for t in model_tensors(model)))
        roof = roofline_tensor(2.0 * w * B / (blk["ms_per_step"] * 1e-3) / 1e12, tf_sus, tf_burst, peak_src, "gemm_tc_kernel",
                               roof["algorithmic_bytes"], TRAFFIC_RATIO["gemm_tc_kernel"])
        roof["note"] = "projection flops over the time of the WHOLE step"
    line = {
        "metric": "tok/s", "value": blk["value"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": blk["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 weights (split12), fp32 accumulate, int8 KV cache",
        "data": "synthetic: seeded N(0,0.02) bf16 weights packed to split12 on the device; random embeddings, norms, tokens "
                "and a random int8 KV cache of `position` entries",
        "config": {"workload": args.workload, "what": cfg["desc"], "layers": layers, "batch": B, "parallelism": "single",
                   "position": cfg["position"], "l2": "inputs larger than L2 (packed weights of one step: %.2f GB)" % (roof["algorithmic_bytes"] / 1e9),
                   "launch": "cuda graph" + ("" if args.no_pdl else " + programmatic dependent launch")},
        "roofline": roof, "e2e": blk["e2e"], "gpu_launches": blk["gpu_launches"], "clocks": clocks, "device_status": status,
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, layers, B, seconds=12.0)
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# CPU statement of the path (oracle port), used as the reported baseline and as the reference arm
# ----------------------------------------------------------------------------------------------

def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class CpuStep:
    """One decode step of the CPU statement of the path (lossless unpack + fp32 GEMM, OpenMP over all host threads):
    the projections of a layer are packed once and run `layers` times per step (a layer's packed weights are 0.33 GB at
    the 7B shapes, far beyond the CPU caches), then the output projection.  Bounded: at most `max_seq` of the batch's
    sequences are computed and the time is scaled to the batch."""

    def __init__(self, cfg, layers, B, max_seq=8):
        from oracle import oracle as O
        self.O = O
        self.threads = O.set_num_threads(host_threads())      # launchers export OMP_NUM_THREADS=1 to their ranks
        H, Q, KV, F, V = cfg["hidden"], cfg["q"], cfg["kv"], cfg["ffn"], cfg["vocab"]
        shapes = [(Q, H)] + ([(KV, H), (KV, H), (H, Q)] if KV else []) + ([(F, H), (F, H), (H, F)] if F else [])
        self.Bc = min(B, max_seq)
        self.B, self.layers = B, layers
        self.layer = [(O.pack(O.synth_weights(M, K, 100 + i)), O.synth_acts(self.Bc, K, i)) for i, (M, K) in enumerate(shapes)]
        self.head = (O.pack(O.synth_weights(V, H, 99)), O.synth_acts(self.Bc, H, 99)) if V else None
        self.layer_weights = sum(M * K for M, K in shapes)
        self.step_weights = self.layer_weights * layers + (V * H if V else 0)

    def run_layers(self, n):
        for _ in range(n):
            for p, x in self.layer:
                self.O.cpu_unpack_gemm_f32(p, x)

    def step(self):
        self.run_layers(self.layers)
        if self.head:
            self.O.cpu_unpack_gemm_f32(*self.head)


def cpu_baseline(cfg, layers, B, seconds=12.0):
    """A bounded sample of the workload on the host cores: whole layers for about `seconds`, scaled to a step."""
    cs = CpuStep(cfg, layers, B)
    cs.run_layers(1)
    n, t0 = 0, time.perf_counter()
    while n < 2 or (time.perf_counter() - t0 < seconds and n < 400):
        cs.run_layers(1)
        n += 1
    per_layer = (time.perf_counter() - t0) / n
    step_s = per_layer * (cs.step_weights / cs.layer_weights) * (B / cs.Bc)
    return {"value": round(B / step_s, 4), "unit": "tok/s", "cores": cs.threads, "kind": "port",
            "sample": f"{n} passes over one layer's projections ({cs.layer_weights / 1e6:.0f} M weights, {cs.Bc} of {B} sequences) in "
                      f"{per_layer * n:.1f} s, mean pass scaled by weight count and batch to a whole step",
            "compressed_GBps": round(cs.layer_weights * 1.5 / per_layer / 1e9, 2)}


def run_reference(args):
    """The CPU statement of the path timed as the arm's own steps: W warm-up steps, then exactly K whole steps."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = WORKLOADS[args.workload]
    layers = args.layers or cfg["layers"]
    B = cfg["batch"]
    t_all = time.perf_counter()
    cs = CpuStep(cfg, layers, B)
    for _ in range(max(args.warmup, 0)):
        cs.step()
    t0 = time.perf_counter()
    for _ in range(max(args.steps, 1)):
        cs.step()
    timed_s = time.perf_counter() - t0
    step_s = timed_s / max(args.steps, 1) * (B / cs.Bc)
    value = round(B / step_s, 4)
    cb = {"value": value, "unit": "tok/s", "cores": cs.threads, "kind": "port",
          "sample": f"{args.steps} whole steps ({layers} passes over one layer's packed projections + the output projection, "
                    f"{cs.step_weights / 1e9:.2f} G weights per step, {cs.Bc} of {B} sequences) timed in {timed_s:.1f} s"
                    + ("" if cs.Bc == B else f", scaled by {B // cs.Bc} to the batch"),
          "compressed_GBps": round(cs.step_weights * 1.5 * max(args.steps, 1) / timed_s / 1e9, 2)}
    line = {
        "impl": "reference", "metric": "tok/s", "value": value, "unit": "tok/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(1e3 * timed_s / max(args.steps, 1), 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp32 (CPU)", "data": "synthetic: seeded N(0,0.02) bf16 weights packed to split12",
        "config": {"workload": args.workload, "what": cfg["desc"], "layers": layers, "batch": B,
                   "note": "the reference has no CPU unpack or GEMM; this is the CPU restatement of its device "
                           "arithmetic (oracle/split12_oracle.c) on all host threads; ms_per_step is the measured time of "
                           "one step of the sample (the sequences computed), value is scaled to the batch"},
        "cpu_baseline": cb,
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "timed_s": round(timed_s, 2), "wall_s": round(time.perf_counter() - t_all, 2),
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    elif WORKLOADS[a.workload].get("full"):
        run_full(a)
    else:
        run_ours(a)
