"""Load-time path on the device: the native tensor loader, the escape table / row list kernels and the
model-directory loader, against the host builder of the library, the oracle's packer and a numpy
forward pass.  Bit-exact for everything that is integer or byte work."""
import ctypes as C
import importlib.util
import os
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

@pytest.fixture(scope="module")
def lib():
    from turbo_lossless_b200 import capi
    return capi.load()


SUFFIXES = ("sm", "gr", "row_off", "patch_cols", "patch_correct", "patch_wrong")


def write_tensor(d, prefix, p, with_base_exp=True):
    """One packed tensor in the converter's file family (engine/convert_model.py:127-134)."""
    for suffix, arr in zip(SUFFIXES, (p.sm, p.gr, p.row_off, p.cols, p.correct, p.wrong)):
        np.ascontiguousarray(arr).tofile(os.path.join(d, f"{prefix}.{suffix}.bin"))
    with open(os.path.join(d, f"{prefix}.dims"), "w") as f:
        f.write(f"{p.M} {p.K} {p.num_patches}" + (f" {p.base_exp}" if with_base_exp else ""))


def host_table(lib, p, counts=True):
    M, n = p.M, p.num_patches
    rb, cn, vals, ne = np.zeros(M, np.int32), np.zeros(M * 256, np.uint8), np.zeros(max(n, 1), np.int16), np.zeros(M, np.int32)
    nne = lib.s12_host_build_escape_table(p.row_off.ctypes.data, p.cols.ctypes.data, p.correct.ctypes.data, M,
                                          rb.ctypes.data, cn.ctypes.data if counts else None, vals.ctypes.data, ne.ctypes.data)
    return rb, cn, vals[:n], ne[:nne]


@pytest.mark.parametrize("M,K,frac", [(8, 64, 5e-2), (300, 512, 2e-2), (4096, 1024, 1e-3), (1031, 2048, 0.2), (64, 128, 0.0)])
def test_device_escape_table_equals_host_builder(lib, O, M, K, frac):
    import torch
    from turbo_lossless_b200 import CompressedWeight
    p = O.pack(O.synth_weights(M, K, 7 + M, outlier_frac=frac))
    w = CompressedWeight.from_host(p.M, p.K, p.base_exp, p.sm, p.gr, p.row_off, p.cols, p.correct, p.wrong, escape_table=False)
    w.build_escape_table_on_device(escape_counts=True)
    torch.cuda.synchronize()
    if p.num_patches == 0:
        assert w.escape_vals is None and w.num_nonempty_rows == 0
        return
    rb, cn, vals, ne = host_table(lib, p)
    assert np.array_equal(w.escape_row_base.cpu().numpy(), rb)
    assert np.array_equal(w.escape_vals.cpu().numpy(), vals)
    assert np.array_equal(w.escape_counts.cpu().numpy(), cn)
    assert w.num_nonempty_rows == len(ne)
    assert np.array_equal(w.patch_nonempty_rows.cpu().numpy(), ne)


def test_one_long_row_and_many_equal_residues(lib, O):
    """A row whose escapes all share a residue mod 256, and one with more than 255 escapes of one residue
    (the count byte wraps like the engine's cast)."""
    import torch
    from turbo_lossless_b200 import CompressedWeight
    M, K = 3, 256 * 300
    row_off = np.array([0, 300, 300, 305], np.int32)
    cols = np.concatenate([np.arange(300, dtype=np.int32) * 256 + 17, np.array([5, 261, 517, 600, 9000], np.int32)])
    correct = (np.arange(305) * 7 + 1).astype(np.int16)
    class P: pass
    p = P(); p.M, p.K, p.num_patches, p.row_off, p.cols, p.correct = M, K, 305, row_off, cols, correct
    dev = lambda a: torch.from_numpy(a).cuda()  # noqa: E731
    w = CompressedWeight(M=M, K=K, base_exp=100, split_sm=torch.zeros(1, dtype=torch.uint8).cuda(),
                         split_gr=torch.zeros(1, dtype=torch.uint8).cuda(), num_patches=305, row_offsets=dev(row_off),
                         patch_cols=dev(cols), patch_correct=dev(correct), patch_wrong=dev(correct))
    w.build_escape_table_on_device(escape_counts=True)
    rb, cn, vals, ne = host_table(lib, p)
    assert np.array_equal(w.escape_vals.cpu().numpy(), vals)
    assert np.array_equal(w.escape_counts.cpu().numpy(), cn) and cn[17] == 300 % 256
    assert np.array_equal(w.patch_nonempty_rows.cpu().numpy(), ne) and list(ne) == [0, 2]


def test_native_loader_reads_the_on_disk_format(tmp_path, lib, O):
    import torch
    from turbo_lossless_b200 import CompressedWeight, S12Error
    d = str(tmp_path)
    p = O.pack(O.synth_weights(520, 4096, 31, outlier_frac=3e-3))
    write_tensor(d, "layer.0.wq", p)
    w = CompressedWeight.load(d, "layer.0.wq", escape_counts=True)
    assert (w.M, w.K, w.base_exp, w.num_patches) == (p.M, p.K, p.base_exp, p.num_patches)
    for got, want in ((w.split_sm, p.sm), (w.split_gr, p.gr), (w.row_offsets, p.row_off), (w.patch_cols, p.cols),
                      (w.patch_correct, p.correct), (w.patch_wrong, p.wrong)):
        assert np.array_equal(got.cpu().numpy(), want)
    rb, cn, vals, ne = host_table(lib, p)
    assert np.array_equal(w.escape_vals.cpu().numpy(), vals) and np.array_equal(w.escape_counts.cpu().numpy(), cn)
    assert np.array_equal(w.patch_nonempty_rows.cpu().numpy(), ne)
    # the loaded tensor decompresses to the original bits
    from turbo_lossless_b200 import Split12Engine
    out = Split12Engine().decompress(w)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint16).reshape(p.M, p.K),
                          np.asarray(O.unpack_exact(p)).view(np.uint16).reshape(p.M, p.K))

    # older dims files have no base_exp field: 0, as in the engine
    write_tensor(d, "old", p, with_base_exp=False)
    assert CompressedWeight.load(d, "old").base_exp == 0
    # empty CSR files: the tensor loads without escapes
    write_tensor(d, "nocsr", p)
    for s in SUFFIXES[2:]:
        open(os.path.join(d, f"nocsr.{s}.bin"), "wb").close()
    w0 = CompressedWeight.load(d, "nocsr")
    assert w0.num_patches == 0 and w0.row_offsets is None and w0.patch_nonempty_rows is None
    # a CSR file of the wrong size, a missing payload file and a missing dims file are errors
    write_tensor(d, "bad", p)
    p.cols[:-1].tofile(os.path.join(d, "bad.patch_cols.bin"))
    with pytest.raises(S12Error):
        CompressedWeight.load(d, "bad")
    os.remove(os.path.join(d, "old.gr.bin"))
    with pytest.raises(S12Error):
        CompressedWeight.load(d, "old")
    with pytest.raises(S12Error):
        CompressedWeight.load(d, "absent")


def test_load_model_runs_a_decode_step(tmp_path, O):
    """A synthetic model directory in the converter's layout -> load_model -> one decode step, against the
    numpy forward pass of the decoder test."""
    import torch
    from oracle import step_oracle as S
    from turbo_lossless_b200.loader import load_model, read_config
    spec = importlib.util.spec_from_file_location("decoder_case", os.path.join(os.path.dirname(__file__), "test_gpu_decoder.py"))
    case = importlib.util.module_from_spec(spec); spec.loader.exec_module(case)
    d = str(tmp_path)
    n_embd, n_head, n_kv, n_ff, n_vocab, n_layer = 256, 4, 2, 512, 777, 2
    with open(os.path.join(d, "config.bin"), "wb") as f:
        f.write(struct.pack("<7i2f", n_vocab, n_embd, n_head, n_kv, n_layer, n_ff, 4096, 10000.0, 1e-5))
    rng = np.random.default_rng(11)
    embd = S.f32_to_bf16(rng.standard_normal((n_vocab, n_embd)).astype(np.float32)).reshape(n_vocab, n_embd)
    embd.tofile(os.path.join(d, "tok_embd.bin"))
    norms = {}
    def norm(name, key):
        norms[key] = (1.0 + 0.1 * rng.standard_normal(n_embd)).astype(np.float32)
        norms[key].tofile(os.path.join(d, name))
    norm("output_norm.bin", "output_norm")
    shapes = {"wq": (256, 256), "wk": (128, 256), "wv": (128, 256), "wo": (256, 256), "w_gate": (512, 256),
              "w_up": (512, 256), "w_down": (256, 512)}
    w = {}
    w[("lm_head", 0)] = O.synth_weights(n_vocab, n_embd, 998, std=0.06, outlier_frac=1e-3)
    write_tensor(d, "output_proj", O.pack(w[("lm_head", 0)]))
    for li in range(n_layer):
        norm(f"layer.{li}.attn_norm.bin", f"attn_norm.{li}")
        norm(f"layer.{li}.ffn_norm.bin", f"ffn_norm.{li}")
        for i, (nm, (M, K)) in enumerate(shapes.items()):
            w[(nm, li)] = O.synth_weights(M, K, 300 * li + i, std=0.06, outlier_frac=1e-3)
            write_tensor(d, f"layer.{li}.{nm}", O.pack(w[(nm, li)]))
    assert read_config(d)["n_ff"] == n_ff
    batch = 2
    dec = load_model(d, batch=batch, max_seq=16, escape_table=True)
    assert dec.cfg.n_vocab == n_vocab and dec.cfg.max_seq == 16 and dec.layers[1]["w_down"].escape_vals is not None
    ref = case.NumpyDecoder(O, S, dec.cfg, w, embd, norms, batch)
    toks, pos = np.array([3, 500], np.int32), np.array([0, 1], np.int32)
    for step in range(3):
        dec.tokens.copy_(torch.from_numpy(toks)); dec.positions.copy_(torch.from_numpy(pos))
        dec.forward()
        torch.cuda.synchronize()
        got, want = dec.logits.cpu().numpy(), ref.forward(toks, pos)
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max(), f"step {step}"
        toks, pos = np.argmax(want, axis=1).astype(np.int32), pos + 1
    with pytest.raises(FileNotFoundError):
        load_model(os.path.join(d, "nowhere"))
