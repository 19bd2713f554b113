#!/usr/bin/env python3
"""Generates tests/golden/converted_tiny/: a tiny model directory written by the REFERENCE's own converter.

Run in a container that holds the reference checkout (REF, default /root/reference) and has `make -C oracle ref`
done.  The script
  1. writes a small Llama-style checkpoint (config.json + one safetensors file, seeded bf16 weights with a few
     x100 outliers so that every tensor has escapes) into a temporary directory,
  2. builds a temporary tree of symlinks  <tmp>/engine/convert_model.py -> REF/engine/convert_model.py  and
     <tmp>/split12_pack.so -> oracle/_ref/split12_pack_ref.so  (the converter loads the packer from its parent
     directory; nothing is written into the reference),
  3. runs the unmodified converter on it and copies its output here,
  4. stores the source tensors' bf16 bit patterns next to it (converted_tiny_source.npz), so that tests can check
     that what the loader brings back is bit for bit what went in.
Nothing here is needed at test time except the two outputs.
"""
import json
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np
import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
REF = os.environ.get("REF", "/root/reference")

CFG = dict(hidden_size=64, num_attention_heads=2, num_key_value_heads=1, num_hidden_layers=2, intermediate_size=128,
           vocab_size=128, max_position_embeddings=2048, rope_theta=10000.0, rms_norm_eps=1e-5)


def tensors():
    g = torch.Generator().manual_seed(20240607)
    H, F, V = CFG["hidden_size"], CFG["intermediate_size"], CFG["vocab_size"]
    kv = H // CFG["num_attention_heads"] * CFG["num_key_value_heads"]

    def w(m, k, std=0.06):
        t = torch.randn(m, k, generator=g) * std
        mask = torch.rand(m, k, generator=g) < 4e-3
        return torch.where(mask, t * 100.0, t).to(torch.bfloat16)

    out = {"model.embed_tokens.weight": torch.randn(V, H, generator=g).to(torch.bfloat16),
           "model.norm.weight": (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16),
           "lm_head.weight": w(V, H)}
    for i in range(CFG["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
        out[p + "post_attention_layernorm.weight"] = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
        out[p + "self_attn.q_proj.weight"] = w(H, H)
        out[p + "self_attn.k_proj.weight"] = w(kv, H)
        out[p + "self_attn.v_proj.weight"] = w(kv, H)
        out[p + "self_attn.o_proj.weight"] = w(H, H)
        out[p + "mlp.gate_proj.weight"] = w(F, H)
        out[p + "mlp.up_proj.weight"] = w(F, H)
        out[p + "mlp.down_proj.weight"] = w(H, F)
    return out


def main():
    packer = os.path.join(ROOT, "oracle", "_ref", "split12_pack_ref.so")
    conv = os.path.join(REF, "engine", "convert_model.py")
    assert os.path.exists(packer), "run `make -C oracle ref` first"
    assert os.path.exists(conv), f"no reference checkout at {REF}"
    src = tensors()
    with tempfile.TemporaryDirectory() as tmp:
        model = os.path.join(tmp, "model")
        os.makedirs(model)
        with open(os.path.join(model, "config.json"), "w") as f:
            json.dump(CFG, f)
        save_file(src, os.path.join(model, "model.safetensors"))
        os.makedirs(os.path.join(tmp, "tree", "engine"))
        os.symlink(conv, os.path.join(tmp, "tree", "engine", "convert_model.py"))
        os.symlink(packer, os.path.join(tmp, "tree", "split12_pack.so"))
        out = os.path.join(tmp, "out")
        subprocess.run([sys.executable, os.path.join(tmp, "tree", "engine", "convert_model.py"), model, out], check=True)
        dst = os.path.join(HERE, "converted_tiny")
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(out, dst)
    np.savez_compressed(os.path.join(HERE, "converted_tiny_source.npz"),
                        **{k: v.contiguous().view(torch.int16).numpy().view(np.uint16) for k, v in src.items()},
                        config=np.frombuffer(json.dumps(CFG).encode(), dtype=np.uint8))
    n = sum(os.path.getsize(os.path.join(dst, f)) for f in os.listdir(dst))
    print(f"wrote {len(os.listdir(dst))} files, {n} bytes, to {dst}")


if __name__ == "__main__":
    main()
