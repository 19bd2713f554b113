"""A minimal decode step around the split12 projections, mirroring the engine's forward loop.

Follows ``forward_b1`` / ``forward_batch_tiled`` of engine/inference.cpp (198-366, 572-666): embed,
RMSNorm -> bf16, q/k/v, RoPE + INT8 KV store, attention over the cache, o, add + RMSNorm, gate/up,
SiLU*up, down, add + RMSNorm of the next layer, ..., lm_head, argmax.  Every operation is one
launch of the CUDA library through its C ABI (the engine's own launcher names); torch only owns
the buffers.  Differences from the engine's loop, all inside the library's documented surface:
q/k/v and gate/up are one launch each with the escapes folded in (``s12_gemv_async`` /
``s12_gemm_multi_async``), and positions live in device memory (the batched RoPE / store / attention
entry points with one cache per sequence), so one captured CUDA graph serves every step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .engine import CompressedWeight, Split12Engine


@dataclass
class DecoderConfig:
    n_embd: int
    n_head: int
    n_head_kv: int
    n_ff: int
    n_vocab: int
    n_layer: int
    max_seq: int = 512
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def kv_dim(self) -> int:
        return self.n_head_kv * self.head_dim


class Decoder:
    """Weights + KV cache + scratch of one model instance for ``batch`` concurrent sequences."""

    def __init__(self, cfg: DecoderConfig, layers: List[Dict[str, CompressedWeight]], lm_head: CompressedWeight,
                 token_embd: torch.Tensor, norms: Dict[str, torch.Tensor], batch: int = 1, eng: Optional[Split12Engine] = None):
        self.cfg, self.layers, self.lm_head, self.token_embd, self.norms = cfg, layers, lm_head, token_embd, norms
        self.B = batch
        self.eng = eng or Split12Engine()
        dev = token_embd.device
        n, hd, B = cfg.n_embd, cfg.head_dim, batch
        f32 = dict(device=dev, dtype=torch.float32)
        self.hidden = torch.zeros(B, n, **f32)
        self.hidden2 = torch.zeros(B, n, **f32)
        self.q_buf = torch.zeros(B, cfg.n_head * hd, **f32)
        self.k_buf = torch.zeros(B, cfg.kv_dim, **f32)
        self.v_buf = torch.zeros(B, cfg.kv_dim, **f32)
        self.ffn_gate = torch.zeros(B, cfg.n_ff, **f32)
        self.ffn_up = torch.zeros(B, cfg.n_ff, **f32)
        self.logits = torch.zeros(B, cfg.n_vocab, **f32)
        assert cfg.n_head * hd == n, "the attention output feeds the o projection: n_head * head_dim must equal n_embd"
        self.bf16_a = torch.zeros(B, n, device=dev, dtype=torch.int16)
        self.bf16_b = torch.zeros(B, cfg.n_ff, device=dev, dtype=torch.int16)
        self.tokens = torch.zeros(B, device=dev, dtype=torch.int32)
        self.next_tokens = torch.zeros(B, device=dev, dtype=torch.int32)
        self.positions = torch.zeros(B, device=dev, dtype=torch.int32)
        # INT8 cache [layer][sequence][position][kv head][head_dim], one fp32 scale per (position, kv head)
        self.kv_stride = cfg.max_seq * cfg.kv_dim
        self.kv_k = torch.zeros(cfg.n_layer, B, cfg.max_seq, cfg.n_head_kv, hd, device=dev, dtype=torch.int8)
        self.kv_v = torch.zeros_like(self.kv_k)
        self.sc_k = torch.zeros(cfg.n_layer, B, cfg.max_seq, cfg.n_head_kv, **f32)
        self.sc_v = torch.zeros_like(self.sc_k)

    # one projection launch: GEMV family for B <= 16, tensor-core GEMM above
    def _proj(self, ws, x_bf16, outs):
        if self.B == 1:
            self.eng.gemv(ws, x_bf16, outs)
        elif len(ws) == 1 and self.B <= 16:
            self.eng.gemv_batched(ws[0], x_bf16, outs[0], x_bf16.stride(0), outs[0].stride(0), self.B)
        else:
            self.eng.gemm_multi(ws, x_bf16, outs, x_bf16.stride(0), self.B)

    def forward(self, attn_len: Optional[int] = None) -> None:
        """One decode step for every sequence: reads ``tokens`` and ``positions`` (device), writes ``logits``
        and ``next_tokens``.  ``attn_len`` = largest position + 1 (sizes the attention's shared memory);
        default: the cache length, which keeps a captured graph valid for every later step."""
        c, e, B = self.cfg, self.eng, self.B
        n, hd = c.n_embd, c.head_dim
        attn_len = attn_len or c.max_seq
        scale = 1.0 / float(hd) ** 0.5
        cur, res = self.hidden, self.hidden2
        e.embed_lookup(self.token_embd, self.tokens, cur)
        for li, L in enumerate(self.layers):
            if li == 0:
                e.rms_norm_bf16(cur, self.norms[f"attn_norm.{li}"], self.bf16_a, c.rms_norm_eps, B)
            if B <= 16 and B > 1:
                for w, o in ((L["wq"], self.q_buf), (L["wk"], self.k_buf), (L["wv"], self.v_buf)):
                    self._proj([w], self.bf16_a, [o])
            else:
                self._proj([L["wq"], L["wk"], L["wv"]], self.bf16_a, [self.q_buf, self.k_buf, self.v_buf])
            e.rope_store_kv_batch(self.q_buf, self.k_buf, self.v_buf, self.kv_k[li], self.kv_v[li], self.sc_k[li], self.sc_v[li],
                                  self.positions, hd, c.n_head, c.n_head_kv, self.kv_stride, c.rope_theta, B)
            e.attention_all_heads_batch(self.q_buf, self.kv_k[li], self.kv_v[li], self.sc_k[li], self.sc_v[li], self.bf16_a,
                                        self.positions, c.n_head, c.n_head_kv, hd, attn_len, scale, B, self.kv_stride)
            self._proj([L["wo"]], self.bf16_a, [res])
            e.rms_norm_bf16(res, self.norms[f"ffn_norm.{li}"], self.bf16_a, c.rms_norm_eps, B, residual=cur)
            if B <= 16 and B > 1:
                self._proj([L["w_gate"]], self.bf16_a, [self.ffn_gate])
                self._proj([L["w_up"]], self.bf16_a, [self.ffn_up])
            else:
                self._proj([L["w_gate"], L["w_up"]], self.bf16_a, [self.ffn_gate, self.ffn_up])
            e.silu_mul_bf16(self.ffn_gate, self.ffn_up, self.bf16_b, c.n_ff, B)
            self._proj([L["w_down"]], self.bf16_b, [cur])
            nxt = self.norms[f"attn_norm.{li + 1}"] if li + 1 < len(self.layers) else self.norms["output_norm"]
            e.rms_norm_bf16(cur, nxt, self.bf16_a, c.rms_norm_eps, B, residual=res)
        self._proj([self.lm_head], self.bf16_a, [self.logits])
        e.argmax(self.logits, self.next_tokens)

    def launches_per_step(self) -> int:
        per_layer = 9 if not (1 < self.B <= 16) else 12
        return 1 + 1 + per_layer * len(self.layers) + 2
