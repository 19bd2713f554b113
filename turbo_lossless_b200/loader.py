"""Loads a converted model directory into a :class:`Decoder`.

Mirrors ``load_model`` of engine/model.cpp:165-283: ``config.bin`` (seven int32 + two float32:
n_vocab n_embd n_head n_head_kv n_layer n_ff n_ctx rope_theta rms_eps), ``tok_embd.bin`` (bf16),
``output_norm.bin`` / ``layer.<i>.attn_norm.bin`` / ``layer.<i>.ffn_norm.bin`` (fp32), the packed tensors
``output_proj`` and ``layer.<i>.{wq,wk,wv,wo,w_gate,w_up,w_down}``, then the INT8 KV cache.  The packed
tensors go through the library's native loader (``CompressedWeight.load``); the small files are read
with numpy.  The context length follows the engine's rule: ``TURBO_CTX`` if set, else
min(8192, what the free device memory holds), at least 128 -- here divided by the number of concurrent
sequences, since every sequence has its own cache.
"""
from __future__ import annotations

import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch

from .decoder import Decoder, DecoderConfig
from .engine import CompressedWeight, Split12Engine

_CONFIG = struct.Struct("<7i2f")
LAYER_TENSORS = ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")


def read_config(directory: str) -> dict:
    """Parses ``config.bin``; raises FileNotFoundError with the engine's hint when it is absent."""
    path = os.path.join(directory, "config.bin")
    if not os.path.exists(path) or os.path.getsize(path) < _CONFIG.size:
        raise FileNotFoundError(f"No config.bin found in {directory} (run the converter on the model directory first)")
    with open(path, "rb") as f:
        v = _CONFIG.unpack(f.read(_CONFIG.size))
    keys = ("n_vocab", "n_embd", "n_head", "n_head_kv", "n_layer", "n_ff", "n_ctx", "rope_theta", "rms_norm_eps")
    return dict(zip(keys, v))


def context_length(cfg: dict, batch: int, free_bytes: int, env: Optional[str] = None) -> int:
    """engine/model.cpp:238-258: per token n_layer*n_head_kv*(2*head_dim int8 + 2 fp32 scales); 512 MB are
    kept free when there is that much, else half of what is left."""
    if env:
        return max(128, int(env))
    head_dim = cfg["n_embd"] // cfg["n_head"]
    per_token = cfg["n_layer"] * cfg["n_head_kv"] * (head_dim * 2 + 2 * 4) * max(1, batch)
    budget = free_bytes - (512 << 20) if free_bytes > (512 << 20) else free_bytes // 2
    return max(128, min(8192, budget // per_token))


def _f32(directory: str, name: str, n: int, device) -> Optional[torch.Tensor]:
    path = os.path.join(directory, name)
    if not os.path.exists(path) or os.path.getsize(path) == 0:
        return None
    a = np.fromfile(path, dtype=np.float32)
    if a.size != n:
        raise ValueError(f"{name}: {a.size} values, expected {n}")
    return torch.from_numpy(a).to(device)


def load_model(directory: str, batch: int = 1, max_seq: Optional[int] = None, device="cuda",
               escape_table: bool = False, eng: Optional[Split12Engine] = None) -> Decoder:
    """Reads every file of a converted model and returns a ready :class:`Decoder` for ``batch`` sequences.
    ``escape_table``: also build the batch4/8 escape table and row list of every tensor (on the device)."""
    cfg = read_config(directory)
    dev = torch.device(device)
    embd_path = os.path.join(directory, "tok_embd.bin")
    if not os.path.exists(embd_path):
        raise FileNotFoundError("Missing tok_embd.bin")
    embd = np.fromfile(embd_path, dtype=np.int16)
    if embd.size != cfg["n_vocab"] * cfg["n_embd"]:
        raise ValueError("tok_embd.bin does not match n_vocab x n_embd")
    token_embd = torch.from_numpy(embd.reshape(cfg["n_vocab"], cfg["n_embd"])).to(dev)

    norms: Dict[str, torch.Tensor] = {}
    t = _f32(directory, "output_norm.bin", cfg["n_embd"], dev)
    if t is not None:
        norms["output_norm"] = t
    lm_head = CompressedWeight.load(directory, "output_proj", device=dev, escape_table=escape_table)
    layers: List[Dict[str, CompressedWeight]] = []
    for i in range(cfg["n_layer"]):
        for kind in ("attn_norm", "ffn_norm"):
            t = _f32(directory, f"layer.{i}.{kind}.bin", cfg["n_embd"], dev)
            if t is not None:
                norms[f"{kind}.{i}"] = t
        layers.append({name: CompressedWeight.load(directory, f"layer.{i}.{name}", device=dev, escape_table=escape_table)
                       for name in LAYER_TENSORS})
    if max_seq is None:
        free = torch.cuda.mem_get_info(dev)[0] if dev.type == "cuda" else 1 << 30
        max_seq = context_length(cfg, batch, free, os.environ.get("TURBO_CTX"))
    dcfg = DecoderConfig(n_embd=cfg["n_embd"], n_head=cfg["n_head"], n_head_kv=cfg["n_head_kv"], n_ff=cfg["n_ff"],
                         n_vocab=cfg["n_vocab"], n_layer=cfg["n_layer"], max_seq=int(max_seq),
                         rms_norm_eps=cfg["rms_norm_eps"], rope_theta=cfg["rope_theta"])
    return Decoder(dcfg, layers, lm_head, token_embd, norms, batch=batch, eng=eng)
