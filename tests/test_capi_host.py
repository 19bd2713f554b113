"""The shared library loads, exports every declared symbol, and its host helpers match the oracle.
No device work is launched here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    from turbo_lossless_b200 import capi
    return capi.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "split12_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(?:int|int64_t|const char\*)\s+(\w+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from turbo_lossless_b200 import capi
    declared = _declared_symbols()
    assert len(declared) >= 24
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == declared


def test_version_and_error_text(lib):
    assert lib.s12_version() >= 100
    assert isinstance(lib.s12_last_error(), bytes)


def test_struct_layouts():
    from turbo_lossless_b200.capi import S12PatchBatchDesc, S12Tensor
    assert C.sizeof(S12PatchBatchDesc) == 56          # "must match PatchBatchDesc exactly"
    assert C.sizeof(S12Tensor) == 6 * 8 + 4 * 4


def _tensor(p):
    from turbo_lossless_b200.capi import S12Tensor
    t = S12Tensor()
    t.sm, t.gr = p.sm.ctypes.data, p.gr.ctypes.data
    t.row_off, t.cols = p.row_off.ctypes.data, p.cols.ctypes.data
    t.correct, t.wrong = p.correct.ctypes.data, p.wrong.ctypes.data
    t.M, t.K, t.base_exp, t.num_patches = p.M, p.K, p.base_exp, p.num_patches
    return t


def test_host_escape_table_matches_oracle(lib, O):
    w = O.synth_weights(50, 768, 21, outlier_frac=2e-2)
    p = O.pack(w)
    rb_o, cnt_o, vals_o, ne_o = O.build_escape_table(p)
    rb = np.zeros(p.M, np.int32); cnt = np.zeros(p.M * 256, np.uint8)
    vals = np.zeros(p.num_patches, np.int16); ne = np.zeros(p.M, np.int32)
    n = lib.s12_host_build_escape_table(p.row_off.ctypes.data, p.cols.ctypes.data, p.correct.ctypes.data,
                                        p.M, rb.ctypes.data, cnt.ctypes.data, vals.ctypes.data, ne.ctypes.data)
    assert n == len(ne_o)
    assert np.array_equal(rb, rb_o) and np.array_equal(cnt, cnt_o)
    assert np.array_equal(vals, vals_o) and np.array_equal(ne[:n], ne_o)
    # counts are optional
    n2 = lib.s12_host_build_escape_table(p.row_off.ctypes.data, p.cols.ctypes.data, p.correct.ctypes.data,
                                         p.M, rb.ctypes.data, None, vals.ctypes.data, ne.ctypes.data)
    assert n2 == n and np.array_equal(vals, vals_o)


@pytest.mark.parametrize("parts", [2, 8])
def test_host_sharders_match_oracle(lib, O, parts):
    w = O.synth_weights(64, 512, 22, outlier_frac=1e-2)
    p = O.pack(w)
    t = _tensor(p)
    cap = max(p.num_patches, 1)
    for i in range(parts):
        for kind in ("rows", "cols"):
            if kind == "rows":
                a, b = i * p.M // parts, (i + 1) * p.M // parts
                exp = O.shard_rows(p, a, b); Ms, Ks = b - a, p.K
                fn = lib.s12_host_shard_rows
            else:
                a, b = i * p.K // parts, (i + 1) * p.K // parts
                exp = O.shard_cols(p, a, b); Ms, Ks = p.M, b - a
                fn = lib.s12_host_shard_cols
            sm = np.zeros(Ms * Ks, np.uint8); gr = np.zeros(Ms * Ks // 2, np.uint8)
            ro = np.zeros(Ms + 1, np.int32); co = np.zeros(cap, np.int32)
            cv = np.zeros(cap, np.int16); wv = np.zeros(cap, np.int16)
            n = fn(C.byref(t), a, b, sm.ctypes.data, gr.ctypes.data, ro.ctypes.data, co.ctypes.data,
                   cv.ctypes.data, wv.ctypes.data)
            assert n == exp.num_patches
            assert np.array_equal(sm, exp.sm) and np.array_equal(gr, exp.gr) and np.array_equal(ro, exp.row_off)
            assert np.array_equal(co[:n], exp.cols) and np.array_equal(cv[:n], exp.correct)
            assert np.array_equal(wv[:n], exp.wrong)


def test_host_sharder_rejects_odd_cuts(lib, O):
    p = O.pack(O.synth_weights(4, 64, 23))
    t = _tensor(p)
    z = np.zeros(4 * 64, np.uint8); ro = np.zeros(5, np.int32)
    assert lib.s12_host_shard_cols(C.byref(t), 1, 33, z.ctypes.data, z.ctypes.data, ro.ctypes.data,
                                   None, None, None) < 0
    assert lib.s12_host_shard_rows(C.byref(t), 2, 9, z.ctypes.data, z.ctypes.data, ro.ctypes.data,
                                   None, None, None) < 0


def test_loader_reads_the_on_disk_format(tmp_path, O):
    """CompressedWeight.from_dir reads the per-tensor file family of engine/convert_model.py:127-134
    (device upload is not exercised here: parsing and validation only)."""
    from turbo_lossless_b200.engine import CompressedWeight
    p = O.pack(O.synth_weights(8, 64, 24, outlier_frac=5e-2))
    d = str(tmp_path)
    for suffix, arr in (("sm", p.sm), ("gr", p.gr), ("row_off", p.row_off), ("patch_cols", p.cols),
                        ("patch_correct", p.correct), ("patch_wrong", p.wrong)):
        arr.tofile(os.path.join(d, f"layer.0.wq.{suffix}.bin"))
    with open(os.path.join(d, "layer.0.wq.dims"), "w") as f:
        f.write(f"{p.M} {p.K} {p.num_patches} {p.base_exp}")
    w = CompressedWeight.from_dir(d, "layer.0.wq", device="cpu")
    assert (w.M, w.K, w.base_exp, w.num_patches) == (p.M, p.K, p.base_exp, p.num_patches)
    assert np.array_equal(w.split_sm.numpy(), p.sm) and np.array_equal(w.patch_cols.numpy(), p.cols)
    assert w.num_nonempty_rows == int(np.count_nonzero(np.diff(p.row_off)))
    os.remove(os.path.join(d, "layer.0.wq.gr.bin"))
    with pytest.raises(FileNotFoundError):
        CompressedWeight.from_dir(d, "layer.0.wq", device="cpu")


def test_model_config_and_context_length(tmp_path):
    """config.bin layout and the context-length rule of engine/model.cpp:181-258."""
    import struct
    from turbo_lossless_b200.loader import context_length, read_config
    with open(tmp_path / "config.bin", "wb") as f:
        f.write(struct.pack("<7i2f", 32000, 4096, 32, 8, 32, 14336, 32768, 1e6, 1e-5))
    cfg = read_config(str(tmp_path))
    assert (cfg["n_vocab"], cfg["n_embd"], cfg["n_head"], cfg["n_head_kv"], cfg["n_layer"], cfg["n_ff"], cfg["n_ctx"]) == \
        (32000, 4096, 32, 8, 32, 14336, 32768)
    assert cfg["rope_theta"] == 1e6 and abs(cfg["rms_norm_eps"] - 1e-5) < 1e-12
    per_token = 32 * 8 * (128 * 2 + 8)
    assert context_length(cfg, 1, 100 << 30) == 8192                       # capped by the default
    assert context_length(cfg, 1, (512 << 20) + 1000 * per_token) == 1000  # capped by free memory less 512 MB
    assert context_length(cfg, 4, (512 << 20) + 4000 * per_token) == 1000  # every sequence has its own cache
    assert context_length(cfg, 1, 100 * per_token) == 128                  # never below 128
    assert context_length(cfg, 1, 1 << 40, env="300") == 300 and context_length(cfg, 1, 1 << 40, env="5") == 128
    with pytest.raises(FileNotFoundError):
        read_config(str(tmp_path / "missing"))
