"""Regenerates tests/golden/split12_pack_golden.npz from the UNMODIFIED reference packer.

Run in a container that has the upstream checkout (the oracle Makefile compiles
its split12_pack.c into oracle/_ref/split12_pack_ref.so):

    make -C oracle && python tests/golden/make_golden.py

Every case stores the bf16 input bits and everything pack_split12 /
split12_find_base_exp returned for it, driven through ctypes exactly as
engine/convert_model.py:97-124 drives them.  The large benchmark tensor
(4096x4096, config 1) is stored as SHA-256 digests of the same outputs.
"""
import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from oracle import oracle as O  # noqa: E402


def cases():
    rng = np.random.default_rng(1234)
    out = {}
    out["tiny_2x64"] = O.synth_weights(2, 64, 1)
    out["odd_rows_5x130"] = O.synth_weights(5, 130, 2, outlier_frac=0.02)
    out["outliers_64x256"] = O.synth_weights(64, 256, 3, outlier_frac=5e-3)
    # every exponent 0..255 appears: most elements escape, several rows are all-escape
    wide = rng.integers(0, 1 << 16, size=(16, 128), dtype=np.uint16)
    out["wide_exponents_16x128"] = wide
    # all exponents inside one 15-wide window: zero escapes, empty CSR arrays
    e = rng.integers(110, 125, size=(8, 96)).astype(np.uint16)
    m = rng.integers(0, 128, size=(8, 96)).astype(np.uint16)
    s = rng.integers(0, 2, size=(8, 96)).astype(np.uint16)
    out["no_escapes_8x96"] = (s << 15) | (e << 7) | m
    # escapes exactly in the first and last column of some rows
    edge = O.synth_weights(12, 64, 4)
    edge[0, 0] = 0x7F80          # +inf
    edge[0, 63] = 0x0000         # zero
    edge[5, 63] = 0xFF81         # NaN
    edge[11, 0] = 0x0001         # denormal
    out["edge_columns_12x64"] = edge
    # window starting at exponent 0 -> base_exp = -1 (zeros and denormals dominate)
    tinyv = rng.integers(0, 1 << 10, size=(6, 64), dtype=np.uint16)   # exponents 0..7
    tinyv[2, 5] = 0x3F80
    out["base_exp_minus1_6x64"] = tinyv
    return out


def main():
    assert O.have_ref_packer(), "oracle/_ref/split12_pack_ref.so missing: run make -C oracle next to the reference"
    blob = {}
    for name, w in cases().items():
        p = O.pack(w, use_ref=True)
        blob[name + ".w"] = w
        blob[name + ".base_exp"] = np.int32(p.base_exp)
        for f in ("sm", "gr", "row_off", "cols", "correct", "wrong"):
            blob[name + "." + f] = getattr(p, f)
        print(f"{name}: M={p.M} K={p.K} base_exp={p.base_exp} escapes={p.num_patches}")
    # config 1 of the benchmark: digests only
    w = O.synth_weights(4096, 4096, 0, outlier_frac=5e-4)
    p = O.pack(w, use_ref=True)
    dig = [hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
           for a in (w, p.sm, p.gr, p.row_off, p.cols, p.correct, p.wrong)]
    blob["config1.digests"] = np.array(dig)
    blob["config1.meta"] = np.array([p.base_exp, p.num_patches], np.int64)
    print(f"config1: base_exp={p.base_exp} escapes={p.num_patches}")
    path = os.path.join(os.path.dirname(__file__), "split12_pack_golden.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
