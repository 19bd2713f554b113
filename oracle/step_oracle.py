"""CPU restatement of the engine's decode-step kernels (engine/kernels.hip) in numpy.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's checker
paths; nothing shipped calls it.  Parity unpinned: the reference has no golden vectors or CPU
statement of these kernels, and its HIP/CUDA kernels are not run here; each function below follows
the arithmetic of the cited kernel (fp32 inputs and outputs, accumulation in float64 so that the
tolerance in the tests is about the kernels' rounding, not the oracle's).
"""
from __future__ import annotations

import numpy as np


def bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    """engine/kernels.hip:16-20"""
    return (raw.astype(np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even on the raw bits, engine/kernels.hip:22-28."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return (r & 0xFFFF).astype(np.uint16).view(np.int16)


def embed_lookup(table_bf16: np.ndarray, tokens: np.ndarray) -> np.ndarray:
    """engine/kernels.hip:57-73: tokens outside the table give zero rows."""
    n_vocab, n_embd = table_bf16.shape
    out = np.zeros((len(tokens), n_embd), dtype=np.float32)
    for s, t in enumerate(tokens):
        if 0 <= t < n_vocab:
            out[s] = bf16_to_f32(table_bf16[t])
    return out


def rms_norm_bf16(x: np.ndarray, weight: np.ndarray, eps: float, residual: np.ndarray | None = None):
    """engine/kernels.hip:355-393 (and :399-442 with the residual add written back).
    Returns (x after the optional add, bf16 output)."""
    x = x.astype(np.float32)
    if residual is not None:
        x = (x + residual.astype(np.float32)).astype(np.float32)
    ss = (x.astype(np.float64) ** 2).sum(axis=-1, keepdims=True)
    rms = 1.0 / np.sqrt(ss / x.shape[-1] + eps)
    y = (x.astype(np.float64) * rms * weight.astype(np.float64)).astype(np.float32)
    return x, f32_to_bf16(y)


def silu_mul_bf16(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """engine/kernels.hip:447-458"""
    g = gate.astype(np.float64)
    return f32_to_bf16((g / (1.0 + np.exp(-g)) * up.astype(np.float64)).astype(np.float32))


def rope_freqs(head_dim: int, theta: float) -> np.ndarray:
    """engine/kernels.hip:129-135, float arithmetic as on the engine's host."""
    d = np.arange(head_dim // 2, dtype=np.float32)
    return (np.float32(1.0) / np.power(np.float32(theta), (np.float32(2.0) * d / np.float32(head_dim)).astype(np.float32))).astype(np.float32)


def rope(x: np.ndarray, position: int, head_dim: int, theta: float) -> np.ndarray:
    """Rotate-half RoPE on [heads, head_dim], engine/kernels.hip:174-215."""
    half = head_dim // 2
    ang = (np.float32(position) * rope_freqs(head_dim, theta)).astype(np.float64)
    c, s = np.cos(ang), np.sin(ang)
    x = x.reshape(-1, head_dim).astype(np.float64)
    x0, x1 = x[:, :half], x[:, half:]
    return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=1).astype(np.float32)


def quantize_head(v: np.ndarray):
    """One (position, kv head) vector -> (int8 values, scale), engine/kernels.hip:220-303."""
    amax = np.float32(np.abs(v).max()) if v.size else np.float32(0)
    scale = np.float32(amax / np.float32(127.0))
    inv = np.float32(127.0) / amax if amax > 0 else np.float32(0)
    q = np.clip(np.rint(v.astype(np.float32) * inv), -127, 127).astype(np.int8)
    return q, scale


def attention(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, sk: np.ndarray, sv: np.ndarray,
              seq_len: int, n_head: int, n_head_kv: int, head_dim: int, scale: float) -> np.ndarray:
    """Decode attention over the INT8 cache, engine/kernels.hip:499-586.
    q [n_head*head_dim] fp32; caches int8 [max_seq, n_head_kv, head_dim]; scales [max_seq, n_head_kv].
    Returns bf16 [n_head*head_dim]."""
    out = np.zeros(n_head * head_dim, dtype=np.float32)
    g = n_head // n_head_kv
    for h in range(n_head):
        kv = h // g
        qh = q[h * head_dim:(h + 1) * head_dim].astype(np.float64)
        k = k_cache[:seq_len, kv, :].astype(np.float64) * sk[:seq_len, kv].astype(np.float64)[:, None]
        s = (k @ qh) * scale
        p = np.exp(s - s.max())
        p = p / p.sum()
        v = v_cache[:seq_len, kv, :].astype(np.float64) * sv[:seq_len, kv].astype(np.float64)[:, None]
        out[h * head_dim:(h + 1) * head_dim] = (p @ v).astype(np.float32)
    return f32_to_bf16(out)


def argmax_engine(logits: np.ndarray) -> int:
    """Greedy pick with the tie rule of engine/kernels.hip:90-122: 256 threads scan i = tid, tid + 256, ...
    with a strict '>', then a tree that keeps the lower thread on equality."""
    n = len(logits)
    best_v = np.full(256, -np.inf, dtype=np.float32)
    best_i = np.zeros(256, dtype=np.int64)
    for tid in range(min(256, n)):
        col = logits[tid::256]
        if len(col) == 0:
            continue
        m = np.nanmax(col) if not np.all(np.isnan(col)) else -np.inf
        if m > -np.inf:
            j = int(np.argmax(col == m))
            best_v[tid], best_i[tid] = m, tid + 256 * j
    s = 128
    while s > 0:
        for tid in range(s):
            if best_v[tid + s] > best_v[tid]:
                best_v[tid], best_i[tid] = best_v[tid + s], best_i[tid + s]
        s //= 2
    return int(best_i[0])


def moe_route(logits: np.ndarray):
    """Top-2 routing as published for Mixtral-8x7B (the reference engine has no MoE path; parity unpinned):
    per token the two largest router logits, ties to the lower expert; weights = softmax over those two.
    Returns (sel [T,2] int32, weight [T,2] float64).  With a single expert the second choice repeats the
    first with weight 0."""
    T, E = logits.shape
    sel = np.zeros((T, 2), np.int32)
    wt = np.zeros((T, 2), np.float64)
    for t in range(T):
        row = logits[t].astype(np.float64)
        i1 = int(np.argmax(row))                       # first of the maxima
        if E == 1:
            sel[t], wt[t] = (i1, i1), (1.0, 0.0)
            continue
        rest = row.copy(); rest[i1] = -np.inf
        i2 = int(np.argmax(rest))
        w2 = 1.0 / (1.0 + np.exp(row[i1] - row[i2]))
        sel[t], wt[t] = (i1, i2), (1.0 - w2, w2)
    return sel, wt


def moe_ffn(x_bf16: np.ndarray, logits: np.ndarray, experts, matmul) -> np.ndarray:
    """out[t] = sum over the token's two experts of weight * down_e(bf16(silu(gate_e x) * up_e x)), fp32.
    ``experts[e]`` = (gate, up, down) in whatever form ``matmul(W, x_bf16_rows)`` takes; it returns [rows][M]."""
    sel, wt = moe_route(logits)
    T = x_bf16.shape[0]
    out = None
    for t in range(T):
        acc = 0.0
        for k in range(2):
            if wt[t, k] == 0.0:
                continue
            g, u, d = experts[sel[t, k]]
            xr = x_bf16[t:t + 1]
            h = silu_mul_bf16(np.asarray(matmul(g, xr), np.float32), np.asarray(matmul(u, xr), np.float32)).reshape(1, -1)
            acc = acc + wt[t, k] * np.asarray(matmul(d, h), np.float64)[0]
        if out is None:
            out = np.zeros((T, len(acc)), np.float32)
        out[t] = acc
    return out
