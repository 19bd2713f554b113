"""Top-2 mixture-of-experts feed-forward block over split12-packed expert weights (Mixtral-8x7B shape).

The reference engine has no MoE path; this block follows the published Mixtral algorithm (the two largest
router logits per token, softmax over those two, SwiGLU experts) and runs as launches of the CUDA library
only: route -> gather by expert -> gate/up of all experts (grouped launches), SiLU*up, down (grouped) -> combine.  Every expert
works on a dense block of ``capacity`` rows (zero rows above its token count), so nothing depends on a
count read back by the host and the whole block can sit inside a captured CUDA graph.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .capi import check
from .engine import CompressedWeight, Split12Engine, _ptr, _stream


class MoEFeedForward:
    """``experts[e]`` = {"w_gate", "w_up", "w_down"}; ``tokens`` = rows per call; ``capacity`` = rows each expert
    processes (default: ``tokens``, which can never overflow)."""

    def __init__(self, experts: List[Dict[str, CompressedWeight]], tokens: int, capacity: Optional[int] = None,
                 eng: Optional[Split12Engine] = None):
        self.experts, self.T = experts, tokens
        self.E = len(experts)
        self.cap = capacity or tokens
        self.eng = eng or Split12Engine()
        w0 = experts[0]
        self.H, self.F = w0["w_gate"].K, w0["w_gate"].M
        dev = w0["w_gate"].split_sm.device
        i32, f32 = dict(device=dev, dtype=torch.int32), dict(device=dev, dtype=torch.float32)
        self.sel = torch.zeros(tokens, 2, **i32)
        self.weight = torch.zeros(tokens, 2, **f32)
        self.slot = torch.zeros(tokens, 2, **i32)
        self.lists = torch.zeros(self.E, tokens, **i32)
        self.counts = torch.zeros(self.E, **i32)
        self.xe = torch.zeros(self.E, self.cap, self.H, device=dev, dtype=torch.int16)
        self.gate = torch.zeros(self.E, self.cap, self.F, **f32)
        self.up = torch.zeros(self.E, self.cap, self.F, **f32)
        self.he = torch.zeros(self.E, self.cap, self.F, device=dev, dtype=torch.int16)
        self.ye = torch.zeros(self.E, self.cap, self.H, **f32)

    @property
    def launches(self) -> int:
        """Kernel launches of one forward call: route, gather, combine, SiLU*up and the projections -- eight tensors
        per launch on the tensor cores (capacity > 16), one per tensor and 16 rows otherwise."""
        if self.cap > 16:
            return 4 + (2 * self.E + 7) // 8 + (self.E + 7) // 8
        return 4 + 3 * self.E * ((self.cap + 15) // 16)

    def forward(self, x_bf16: torch.Tensor, router_logits: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
                stream=None) -> None:
        """x_bf16 int16 [T][H], router_logits fp32 [T][E], out fp32 [T][H] (added to when ``accumulate``)."""
        lib, e, st = self.eng.lib, self.eng, _stream(stream)
        T, E, cap = self.T, self.E, self.cap
        check(lib.s12_moe_route_async(_ptr(router_logits), T, E, _ptr(self.sel), _ptr(self.weight), _ptr(self.slot),
                                      _ptr(self.lists), _ptr(self.counts), st), "s12_moe_route_async")
        check(lib.s12_moe_gather_async(_ptr(x_bf16), self.H, T, E, cap, _ptr(self.lists), _ptr(self.counts), _ptr(self.xe), st),
              "s12_moe_gather_async")
        # all experts' gate/up as grouped launches (expert i reads rows [i*cap, (i+1)*cap) of xe), one SiLU*up over
        # all blocks, all experts' down projections as grouped launches
        ws, rows, outs = [], [], []
        for i, w in enumerate(self.experts):
            ws += [w["w_gate"], w["w_up"]]; rows += [i * cap, i * cap]; outs += [self.gate[i], self.up[i]]
        e.gemm_grouped(ws, self.xe, rows, outs, self.H, cap, stream=stream)
        e.silu_mul_bf16(self.gate, self.up, self.he, self.F, E * cap, stream=stream)
        e.gemm_grouped([w["w_down"] for w in self.experts], self.he, [i * cap for i in range(E)],
                       [self.ye[i] for i in range(E)], self.F, cap, stream=stream)
        check(lib.s12_moe_combine_async(_ptr(self.ye), self.H, T, cap, _ptr(self.sel), _ptr(self.weight), _ptr(self.slot),
                                        _ptr(out), int(accumulate), st), "s12_moe_combine_async")

