"""A model directory written by the reference's OWN converter (engine/convert_model.py, run unmodified by
tests/golden/make_converted_model.py; committed under tests/golden/converted_tiny) against the source weights it
was made from: the oracle on the CPU, the library's loader and decode step on the GPU."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from conftest import ROOT

FIXTURE = os.path.join(ROOT, "tests", "golden", "converted_tiny")
SOURCE = os.path.join(ROOT, "tests", "golden", "converted_tiny_source.npz")
HF = {"wq": "self_attn.q_proj", "wk": "self_attn.k_proj", "wv": "self_attn.v_proj", "wo": "self_attn.o_proj",
      "w_gate": "mlp.gate_proj", "w_up": "mlp.up_proj", "w_down": "mlp.down_proj"}


@pytest.fixture(scope="module")
def src():
    z = np.load(SOURCE)
    cfg = json.loads(bytes(z["config"]).decode())
    return z, cfg


def _names(cfg):
    yield "output_proj", "lm_head.weight"
    for i in range(cfg["num_hidden_layers"]):
        for ours, hf in HF.items():
            yield f"layer.{i}.{ours}", f"model.layers.{i}.{hf}.weight"


def _read_packed(O, prefix):
    M, K, npatch, base_exp = (int(v) for v in open(os.path.join(FIXTURE, prefix + ".dims")).read().split())
    rd = lambda suffix, dt: np.fromfile(os.path.join(FIXTURE, f"{prefix}.{suffix}.bin"), dtype=dt)  # noqa: E731
    p = O.Packed(M, K, base_exp, rd("sm", np.uint8), rd("gr", np.uint8), rd("row_off", np.int32), rd("patch_cols", np.int32),
                 rd("patch_correct", np.int16), rd("patch_wrong", np.int16))
    assert p.num_patches == npatch
    return p


def test_oracle_unpacks_the_converters_files_to_the_source_weights(O, src):
    z, cfg = src
    escapes = 0
    for prefix, hf in _names(cfg):
        p = _read_packed(O, prefix)
        w = z[hf]
        assert (p.M, p.K) == w.shape
        assert np.array_equal(O.unpack_exact(p), w), prefix                       # lossless
        mine = O.pack(w)                                                           # and the oracle packs the same bytes
        assert mine.base_exp == p.base_exp
        for f in ("sm", "gr", "row_off", "cols", "correct", "wrong"):
            assert np.array_equal(getattr(mine, f), getattr(p, f)), (prefix, f)
        escapes += p.num_patches
    assert escapes > 100                                                           # the fixture exercises the escape lists


def test_library_reads_the_dims_files(src):
    from turbo_lossless_b200 import capi
    lib = capi.load()
    z, cfg = src
    for prefix, hf in _names(cfg):
        M, K, be, npatch = C.c_int(), C.c_int(), C.c_int(), C.c_int64()
        assert lib.s12_tensor_dims(FIXTURE.encode(), prefix.encode(), C.byref(M), C.byref(K), C.byref(npatch), C.byref(be)) == 0
        assert (M.value, K.value) == z[hf].shape
        want = open(os.path.join(FIXTURE, prefix + ".dims")).read().split()
        assert [M.value, K.value, npatch.value, be.value] == [int(v) for v in want]


@pytest.mark.gpu
def test_loader_brings_back_the_source_weights_bit_for_bit(src):
    import torch
    from turbo_lossless_b200 import Split12Engine
    from turbo_lossless_b200.loader import load_model, read_config
    z, cfg = src
    rc = read_config(FIXTURE)
    assert (rc["n_vocab"], rc["n_embd"], rc["n_head"], rc["n_head_kv"], rc["n_layer"], rc["n_ff"], rc["n_ctx"]) == (
        cfg["vocab_size"], cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
        cfg["num_hidden_layers"], cfg["intermediate_size"], cfg["max_position_embeddings"])
    eng = Split12Engine()
    dec = load_model(FIXTURE, batch=1, max_seq=8, escape_table=True, eng=eng)
    assert np.array_equal(dec.token_embd.cpu().numpy().view(np.uint16), z["model.embed_tokens.weight"])
    bf = lambda a: (a.astype(np.uint32) << 16).view(np.float32)                    # noqa: E731
    assert np.array_equal(dec.norms["output_norm"].cpu().numpy(), bf(z["model.norm.weight"]))
    for i in range(cfg["num_hidden_layers"]):
        assert np.array_equal(dec.norms[f"attn_norm.{i}"].cpu().numpy(), bf(z[f"model.layers.{i}.input_layernorm.weight"]))
        assert np.array_equal(dec.norms[f"ffn_norm.{i}"].cpu().numpy(), bf(z[f"model.layers.{i}.post_attention_layernorm.weight"]))
    for prefix, hf in _names(cfg):
        cw = dec.lm_head if prefix == "output_proj" else dec.layers[int(prefix.split(".")[1])][prefix.split(".")[2]]
        got = eng.decompress(cw).cpu().numpy().view(np.uint16).reshape(cw.M, cw.K)
        assert np.array_equal(got, z[hf]), prefix
    assert eng.device_status() == 0


@pytest.mark.gpu
def test_decode_steps_on_the_converted_model(O, src):
    """Three greedy steps of the loaded model against the numpy forward pass over the SOURCE weights."""
    import importlib.util
    import torch
    from oracle import step_oracle as S
    from turbo_lossless_b200.loader import load_model
    spec = importlib.util.spec_from_file_location("decoder_case", os.path.join(ROOT, "tests", "test_gpu_decoder.py"))
    case = importlib.util.module_from_spec(spec); spec.loader.exec_module(case)
    z, cfg = src
    batch = 2
    dec = load_model(FIXTURE, batch=batch, max_seq=16)
    w = {("lm_head", 0): z["lm_head.weight"]}
    norms = {"output_norm": (z["model.norm.weight"].astype(np.uint32) << 16).view(np.float32)}
    for i in range(cfg["num_hidden_layers"]):
        for ours, hf in HF.items():
            w[(ours, i)] = z[f"model.layers.{i}.{hf}.weight"]
        norms[f"attn_norm.{i}"] = (z[f"model.layers.{i}.input_layernorm.weight"].astype(np.uint32) << 16).view(np.float32)
        norms[f"ffn_norm.{i}"] = (z[f"model.layers.{i}.post_attention_layernorm.weight"].astype(np.uint32) << 16).view(np.float32)
    ref = case.NumpyDecoder(O, S, dec.cfg, w, z["model.embed_tokens.weight"], norms, batch)
    toks, pos = np.array([3, 100], np.int32), np.array([0, 1], np.int32)
    for step in range(3):
        dec.tokens.copy_(torch.from_numpy(toks)); dec.positions.copy_(torch.from_numpy(pos))
        dec.forward()
        torch.cuda.synchronize()
        got, want = dec.logits.cpu().numpy(), ref.forward(toks, pos)
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max(), f"step {step}"
        toks, pos = np.argmax(want, axis=1).astype(np.int32), pos + 1
