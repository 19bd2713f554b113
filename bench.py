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

With N > 1 (under torchrun) the projections are tensor-parallel: q/k/v, gate/up
and the output projection are split by rows, o and down by columns with an NCCL
all-reduce of the fp32 result after each.
"""
from __future__ import annotations

import argparse
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


# (dram read + write) / packed bytes measured with ncu, per dominant kernel
TRAFFIC_RATIO = {"gemv_stream_kernel": 1.022, "gemm_tc_kernel": 1.154}


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
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (development only)")
    ap.add_argument("--comm", default="own", choices=["own", "fused", "nccl"],
                    help="all-reduce after the row-parallel projections at N > 1: own = this library's one-shot kernel over "
                         "peer memory as a node of the step's CUDA graph (fastest measured: the next GEMV prefetches its "
                         "weights while it runs); fused = the B=1 GEMV pushes its rows to the peers and adds them itself "
                         "(one kernel, but its CTAs stay resident while they wait); nccl = NCCL between graph segments")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops_sustained", p.get("bf16_tflops", 1398.0))), "measured"
    return 6650.0, 1400.0, "fallback"


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
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
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


# ----------------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------------

def build_model(cfg, rank, world, layers, torch, CompressedWeight):
    """Random-init weights of every projection, generated on the device per tensor from a seed that
    depends on (layer, tensor) only, sharded for tensor parallelism and packed by the device packer."""
    dev = torch.device("cuda")
    H, Q, KV, F, V = cfg["hidden"], cfg["q"], cfg["kv"], cfg["ffn"], cfg["vocab"]
    outlier = cfg is WORKLOADS["config1"]

    def make(M, K, seed, split, outlier_frac=5e-4 if outlier else 0.0):
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

    model = {"layers": [], "lm_head": None}
    for layer in range(layers):
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
    layers = args.layers or cfg["layers"]
    B, H, V = cfg["batch"], cfg["hidden"], cfg["vocab"]
    eng = Split12Engine()
    comm = TPComm(rank, world, B * H) if (world > 1 and args.comm != "nccl") else None
    use_fused = comm is not None and args.comm == "fused" and B == 1
    _log("process group up; building model")
    model = build_model(cfg, rank, world, layers, torch, CompressedWeight)
    _log("model packed")
    tensors = model_tensors(model)
    comp_bytes = sum(t.compressed_bytes for t in tensors)             # this rank
    weights = sum(t.M * t.K for t in tensors)
    torch.cuda.synchronize()

    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(7 + rank * 0)
    # activation buffers (bf16) and outputs (fp32); inputs of the row-parallel projections are the
    # rank's column slice
    def act(k):
        return torch.randn(B, k, generator=gen, device=dev).to(torch.bfloat16).view(torch.int16)

    L0 = model["layers"][0]
    x_hidden = act(H)
    x_attn = act(L0["wo"].K) if "wo" in L0 else None
    x_ffn = act(L0["w_down"].K) if "w_down" in L0 else None
    o_q = torch.empty(B, L0["wq"].M, device=dev)
    o_k = torch.empty(B, L0["wk"].M, device=dev) if "wk" in L0 else None
    o_v = torch.empty(B, L0["wv"].M, device=dev) if "wv" in L0 else None
    o_o = torch.empty(B, H, device=dev)
    o_g = torch.empty(B, L0["w_gate"].M, device=dev) if "w_gate" in L0 else None
    o_u = torch.empty(B, L0["w_up"].M, device=dev) if "w_up" in L0 else None
    o_d = torch.empty(B, H, device=dev)
    logits = torch.empty(B, model["lm_head"].M, device=dev) if model["lm_head"] is not None else o_q
    x_host = torch.empty(B, H, dtype=torch.int16).pin_memory()
    x_host.copy_(x_hidden.cpu())
    logits_host = torch.empty(logits.shape, dtype=torch.float32).pin_memory()

    moe_blocks, router_logits = [], None
    if cfg.get("experts"):
        if world > 1:
            raise SystemExit("mixtral_b64 runs on one GPU (expert weights are not sharded)")
        from turbo_lossless_b200.moe import MoEFeedForward
        router_logits = torch.rand(B, cfg["experts"], generator=gen, device=dev)
        moe_blocks = [MoEFeedForward(L["experts"], B, eng=eng) for L in model["layers"]]

    launches = [0]

    def proj(ws, x, outs):
        """One or several tensors sharing an activation: one launch at B=1, one GEMM per tensor else."""
        if B == 1:
            eng.gemv(ws, x, outs)
            launches[0] += 1
        else:
            eng.gemm_multi(ws, x, outs, x.shape[1], B)
            launches[0] += 1

    # The step as a list of segments: ("k", fn) = our launches only (capturable as one CUDA graph),
    # ("ar", tensor) = an NCCL all-reduce after a row-parallel projection.  With --comm own (default) the
    # all-reduce is a kernel of this library and the whole step stays one graph.  NCCL collectives are
    # kept out of graph capture (capturing them hung on this pool), so with --comm nccl a step replays
    # one small graph per segment and calls all_reduce between them.
    segments = []

    def fused(w, x, out):
        """Row-parallel GEMV and the sum over ranks as one kernel (B = 1)."""
        comm.gemv_all_reduce(w, x, out)
        launches[0] += 1

    def all_reduce(t):
        if comm is not None:
            def ar(t=t):
                comm.all_reduce(t)
                launches[0] += 1
            add_k(ar)
        else:
            segments.append(("ar", t))

    def add_k(fn):
        if segments and segments[-1][0] == "k":
            prev = segments[-1][1]
            segments[-1] = ("k", lambda prev=prev, fn=fn: (prev(), fn()))
        else:
            segments.append(("k", fn))

    def moe_layer(L, blk):
        """Attention projections, then the top-2 expert block in place of the dense feed-forward."""
        proj([L["wq"], L["wk"], L["wv"]], x_hidden, [o_q, o_k, o_v])
        proj([L["wo"]], x_attn, [o_o])
        blk.forward(x_hidden, router_logits, o_d)
        launches[0] += blk.launches

    for L, blk in zip(model["layers"], moe_blocks):
        add_k(lambda L=L, blk=blk: moe_layer(L, blk))
    for L in ([] if moe_blocks else model["layers"]):
        if "wk" in L:
            add_k(lambda L=L: proj([L["wq"], L["wk"], L["wv"]], x_hidden, [o_q, o_k, o_v]))
            if use_fused:
                add_k(lambda L=L: fused(L["wo"], x_attn, o_o))
            else:
                add_k(lambda L=L: proj([L["wo"]], x_attn, [o_o]))
                if world > 1:
                    all_reduce(o_o)
        else:
            add_k(lambda L=L: proj([L["wq"]], x_hidden, [o_q]))
        if "w_gate" in L:
            add_k(lambda L=L: proj([L["w_gate"], L["w_up"]], x_hidden, [o_g, o_u]))
            if use_fused:
                add_k(lambda L=L: fused(L["w_down"], x_ffn, o_d))
            else:
                add_k(lambda L=L: proj([L["w_down"]], x_ffn, [o_d]))
                if world > 1:
                    all_reduce(o_d)
    if model["lm_head"] is not None:
        add_k(lambda: proj([model["lm_head"]], x_hidden, [logits]))

    def step():
        for kind, item in segments:
            if kind == "k":
                item()
            else:
                dist.all_reduce(item)

    eng.set_dependent_launch(not args.no_pdl)
    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        step()                                   # also loads every kernel before capture
        torch.cuda.synchronize()
        _log("first eager step done")
        launches_per_step = launches[0]
        if not args.no_graph:
            try:
                graphs = []
                for kind, item in segments:
                    if kind != "k":
                        graphs.append((kind, item))
                        continue
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        item()
                    graphs.append(("g", g))
                graph = graphs
            except Exception as e:               # eager launches still measure the same work
                sys.stderr.write(f"[bench] graph capture failed ({e}); launching eagerly\n")
                graph = None
                torch.cuda.synchronize()

        def replay():
            for kind, item in graph:
                if kind == "g":
                    item.replay()
                else:
                    dist.all_reduce(item)

        run = replay if graph is not None else step
        _log("graph(s) captured: %d segments" % len(graph) if graph is not None else "eager mode")

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        for _ in range(args.warmup):
            run()
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            run()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if rank == 0 else None
        _log(f"timed region done: {ms / args.steps:.3f} ms/step")

        # end to end: pinned host activations in, logits back to the host, every step
        for i in range(2):
            x_hidden.copy_(x_host, non_blocking=True); run(); logits_host.copy_(logits, non_blocking=True)
            if os.environ.get("S12_BENCH_VERBOSE"):
                stream.synchronize()
                _log(f"end-to-end warm-up step {i} done, device status {eng.device_status():#x}")
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            x_hidden.copy_(x_host, non_blocking=True)
            run()
            logits_host.copy_(logits, non_blocking=True)
            stream.synchronize()
        barrier()
        e2e_s = time.perf_counter() - t0

    t = torch.tensor([ms, e2e_s * 1e3], device=dev, dtype=torch.float64)
    tot = torch.tensor([float(comp_bytes), float(weights)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms, e2e_ms = float(t[0]), float(t[1])
    status = eng.device_status()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    hbm_peak, tf_peak, peak_src = peaks()
    ms_step = ms / args.steps
    toks = B * args.steps / (ms / 1e3)
    total_bytes, total_weights = float(tot[0]), float(tot[1])
    per_gpu_gbs = (total_bytes / world) / (ms_step * 1e-3) / 1e9
    if B >= 128:
        achieved = 2.0 * total_weights * B / world / (ms_step * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": round(achieved, 2), "peak": tf_peak, "unit": "TFLOP/s",
                "frac": round(achieved / tf_peak, 4), "traffic": None}
    else:
        roof = {"bound": "hbm", "achieved": round(per_gpu_gbs, 1), "peak": hbm_peak, "unit": "GB/s",
                "frac": round(per_gpu_gbs / hbm_peak, 4), "traffic": None}
    roof["peak_source"] = f"{peak_src} (MEASURED_PEAKS.json)" if peak_src == "measured" else "fallback"
    roof["kernel"] = "gemv_stream_kernel" if B == 1 else ("gemm_tc_kernel" if B > 16 else "gemv_kernel")
    # DRAM bytes (read + write) per step and GPU: ncu captures of a one-layer run of the same workload
    # (summaries under profiles/) gave this ratio to the packed bytes; traffic grows with the layer count.
    ratio = TRAFFIC_RATIO.get(roof["kernel"])
    roof["traffic"] = int(total_bytes / world * ratio) if ratio else None
    roof["traffic_source"] = "ncu dram__bytes_read.sum + dram__bytes_write.sum on a one-layer run, scaled by packed bytes" if ratio else None
    roof["algorithmic_bytes_per_step"] = int(total_bytes)

    line = {
        "metric": "tok/s", "value": round(toks, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 weights (split12), fp32 accumulate",
        "data": "synthetic: seeded N(0,0.02) bf16 weights packed to split12 on the device; random bf16 activations",
        "config": {"workload": args.workload, "what": cfg["desc"], "layers": layers, "batch": B,
                   "parallelism": f"tp{world}" if world > 1 else "single",
                   "collective": ("none" if world == 1 else
                                  ("row-parallel GEMV fused with its one-shot all-reduce over NVLink peer memory (one kernel)" if use_fused
                                   else "one-shot all-reduce kernel over NVLink peer memory, inside the step's graph") if comm is not None
                                  else "NCCL all_reduce between graph segments"),
                   "l2": "inputs larger than L2 (packed weights of one step: %.2f GB per GPU)" % (total_bytes / world / 1e9),
                   "launch": ("cuda graph" if graph is not None else "eager") + ("" if args.no_pdl else " + programmatic dependent launch"),
                   "excluded": "norm/rope/attention/argmax kernels between the projections are not timed here (the *_full workloads time the whole step)"},
        "compressed_GBps_per_gpu": round(per_gpu_gbs, 1),
        "roofline": roof,
        "e2e": {"value": round(B * args.steps / e2e_ms * 1e3, 2), "unit": "tok/s",
                "h2d_bytes_per_step": int(x_host.numel() * 2), "d2h_bytes_per_step": int(logits_host.numel() * 4)},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks, "device_status": status,
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, layers, total_weights, B, seconds=12.0)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_full(args):
    """Whole decode step through turbo_lossless_b200.decoder.Decoder, one GPU."""
    import torch
    from turbo_lossless_b200 import CompressedWeight, Decoder, DecoderConfig, Split12Engine
    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"unavailable": "the *_full workloads run on one GPU"}), flush=True)
        return
    torch.cuda.set_device(0)
    cfg = WORKLOADS[args.workload]
    layers = args.layers or cfg["layers"]
    B, H, V = cfg["batch"], cfg["hidden"], cfg["vocab"]
    eng = Split12Engine()
    model = build_model(cfg, 0, 1, layers, torch, CompressedWeight)
    tensors = model_tensors(model)
    total_bytes = float(sum(t.compressed_bytes for t in tensors))
    total_weights = float(sum(t.M * t.K for t in tensors))
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(11)
    dc = DecoderConfig(n_embd=H, n_head=cfg["heads"], n_head_kv=cfg["kv_heads"], n_ff=cfg["ffn"], n_vocab=V, n_layer=layers,
                       max_seq=cfg["max_seq"])
    embd = torch.randn(V, H, generator=gen, device=dev).to(torch.bfloat16).view(torch.int16)
    names = [f"attn_norm.{i}" for i in range(layers)] + [f"ffn_norm.{i}" for i in range(layers)] + ["output_norm"]
    norms = {nm: 1.0 + 0.1 * torch.randn(H, generator=gen, device=dev) for nm in names}
    dec = Decoder(dc, model["layers"], model["lm_head"], embd, norms, batch=B, eng=eng)
    # a cache that looks like `position` earlier steps: random int8 entries and scales of the size real keys give
    pos = cfg["position"]
    dec.kv_k.copy_(torch.randint(-127, 128, dec.kv_k.shape, generator=gen, device=dev, dtype=torch.int8))
    dec.kv_v.copy_(torch.randint(-127, 128, dec.kv_v.shape, generator=gen, device=dev, dtype=torch.int8))
    dec.sc_k.fill_(0.02); dec.sc_v.fill_(0.02)
    dec.positions.fill_(pos)
    tok_host = torch.randint(0, V, (B,), dtype=torch.int32).pin_memory()
    out_host = torch.zeros(B, dtype=torch.int32).pin_memory()
    dec.tokens.copy_(tok_host)
    eng.set_dependent_launch(not args.no_pdl)
    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        dec.forward(attn_len=pos + 1)
        torch.cuda.synchronize()
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                dec.forward(attn_len=pos + 1)
        run = graph.replay if graph is not None else (lambda: dec.forward(attn_len=pos + 1))
        for _ in range(args.warmup):
            run()
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        # end to end: token ids in from pinned host memory, the greedy tokens back, every step
        for _ in range(2):
            dec.tokens.copy_(tok_host, non_blocking=True); run(); out_host.copy_(dec.next_tokens, non_blocking=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            dec.tokens.copy_(tok_host, non_blocking=True)
            run()
            out_host.copy_(dec.next_tokens, non_blocking=True)
            stream.synchronize()
        e2e_s = time.perf_counter() - t0
    status = eng.device_status()
    hbm_peak, tf_peak, peak_src = peaks()
    ms_step = ms / args.steps
    gbs = total_bytes / (ms_step * 1e-3) / 1e9
    if B >= 128:
        achieved = 2.0 * total_weights * B / (ms_step * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": round(achieved, 2), "peak": tf_peak, "unit": "TFLOP/s",
                "frac": round(achieved / tf_peak, 4), "kernel": "gemm_tc_kernel"}
    else:
        roof = {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(gbs / hbm_peak, 4),
                "kernel": "gemv_stream_kernel"}
    ratio = TRAFFIC_RATIO.get(roof["kernel"])
    roof["traffic"] = int(total_bytes * ratio) if ratio else None
    roof["peak_source"] = f"{peak_src} (MEASURED_PEAKS.json)" if peak_src == "measured" else "fallback"
    roof["note"] = "projection bytes / flops over the time of the WHOLE step (attention, norms, ... included in the time only)"
    roof["algorithmic_bytes_per_step"] = int(total_bytes)
    line = {
        "metric": "tok/s", "value": round(B * args.steps / (ms / 1e3), 2), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 weights (split12), fp32 accumulate, int8 KV cache",
        "data": "synthetic: seeded N(0,0.02) bf16 weights packed to split12 on the device; random embeddings, norms, tokens "
                "and a random int8 KV cache of `position` entries",
        "config": {"workload": args.workload, "what": cfg["desc"], "layers": layers, "batch": B, "parallelism": "single",
                   "position": pos, "l2": "inputs larger than L2 (packed weights of one step: %.2f GB)" % (total_bytes / 1e9),
                   "launch": ("cuda graph" if graph is not None else "eager") + ("" if args.no_pdl else " + programmatic dependent launch")},
        "compressed_GBps_per_gpu": round(gbs, 1), "roofline": roof,
        "e2e": {"value": round(B * args.steps / e2e_s, 2), "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
        "gpu_launches": dec.launches_per_step() * args.steps, "clocks": clocks, "device_status": status,
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, layers, total_weights, B, seconds=12.0)
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# CPU statement of the path (oracle port), used as the reported baseline and as the reference arm
# ----------------------------------------------------------------------------------------------

def cpu_baseline(cfg, layers, total_weights, B, seconds=12.0, steps=1, warmup=0):
    """Times the CPU statement of the path (lossless unpack + fp32 GEMM, all host threads) on one
    layer's projections and scales by the weight count to a whole step."""
    from oracle import oracle as O
    H, Q, KV, F = cfg["hidden"], cfg["q"], cfg["kv"], cfg["ffn"]
    shapes = [(Q, H)] + ([(KV, H), (KV, H), (H, Q)] if KV else []) + ([(F, H), (F, H), (H, F)] if F else [])
    Bc = min(B, 8)                                  # bounded: 8 of the B sequences, scaled below
    packs, acts = [], []
    for i, (M, K) in enumerate(shapes):
        w = O.synth_weights(M, K, 100 + i)
        packs.append(O.pack(w))
        acts.append(O.synth_acts(Bc, K, i))
    sample_weights = sum(M * K for M, K in shapes)
    times = []
    t_end = time.perf_counter() + seconds
    n = 0
    while n < warmup + steps or (time.perf_counter() < t_end and n < warmup + 50):
        t0 = time.perf_counter()
        for p, x in zip(packs, acts):
            O.cpu_unpack_gemm_f32(p, x)
        dt = time.perf_counter() - t0
        if n >= warmup:
            times.append(dt)
        n += 1
    best = min(times)
    step_s = best * (total_weights / sample_weights) * (B / Bc)
    return {"value": round(B / step_s, 4), "unit": "tok/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"one layer's projections ({sample_weights / 1e6:.0f} M weights, {Bc} of {B} sequences), best of "
                      f"{len(times)} passes, scaled by weight count and batch to a whole step",
            "compressed_GBps": round(sample_weights * 1.5 / best / 1e9, 2)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = WORKLOADS[args.workload]
    layers = args.layers or cfg["layers"]
    H, Q, KV, F, V = cfg["hidden"], cfg["q"], cfg["kv"], cfg["ffn"], cfg["vocab"]
    per_layer = Q * H + (2 * KV * H + H * Q if KV else 0) + (3 * F * H if F else 0)
    total_weights = per_layer * layers + V * H
    B = cfg["batch"]
    t0 = time.perf_counter()
    cb = cpu_baseline(cfg, layers, total_weights, B, seconds=0.0, steps=max(args.steps, 1), warmup=max(args.warmup, 0))
    line = {
        "impl": "reference", "metric": "tok/s", "value": cb["value"], "unit": "tok/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(1e3 * B / cb["value"], 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp32 (CPU)", "data": "synthetic: seeded N(0,0.02) bf16 weights packed to split12",
        "config": {"workload": args.workload, "what": cfg["desc"], "layers": layers, "batch": B,
                   "note": "the reference has no CPU unpack or GEMM; this is the CPU restatement of its device "
                           "arithmetic (oracle/split12_oracle.c) on all host threads"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": round(time.perf_counter() - t0, 2),
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
