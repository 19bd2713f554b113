"""The numpy statement of the decode-step kernels (oracle/step_oracle.py) and this library's launchers pinned to
the reference's OWN kernels: `make -C oracle ref_step` compiles engine/kernels.hip unmodified (through its
gpu_compat.h) for sm_100a into oracle/_ref/libturbo_ref_step.so; this file runs both libraries on the same
inputs (skipped when that library has not been built).

Only launches whose behaviour was checked by reading the reference are made: rows of 4096 for the norms (its
cross-warp reduction is written for 1024 threads), head_dim 128, at most 384 cached positions (its attention
keeps one score per position in shared memory without raising the 48 KB limit; its flash-attention path asks for
more than that limit and is never run here), RoPE at small positions (it uses the fast sincos intrinsic, this
library the accurate one; both are compared with the float64 oracle at a tolerance that covers the intrinsic).
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libturbo_ref_step.so")
_vp, _i, _f = C.c_void_p, C.c_int, C.c_float


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libturbo_ref_step.so not built (make -C oracle ref_step next to the reference)")
    lib = C.CDLL(REF_LIB)
    sigs = {
        "launch_embed_lookup": [_vp, _vp, _vp, _i, _i, _i, _vp],
        "launch_argmax": [_vp, _vp, _i, _vp],
        "launch_argmax_batch": [_vp, _vp, _i, _i, _vp],
        "launch_rms_norm_bf16_batch": [_vp, _vp, _vp, _i, _f, _i, _vp],
        "launch_add_rms_norm_bf16_batch": [_vp, _vp, _vp, _vp, _i, _f, _i, _vp],
        "launch_silu_mul_bf16_batch": [_vp, _vp, _vp, _i, _i, _vp],
        "launch_add_batch": [_vp, _vp, _i, _i, _vp],
        "launch_rope_store_kv": [_vp] * 7 + [_i, _i, _i, _i, _i, _f, _vp],
        "launch_rope_batch": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp],
        "launch_store_kv_batch": [_vp] * 7 + [_i, _i, _i, _i, _i, _vp],
        "launch_attention_all_heads": [_vp] * 6 + [_i, _i, _i, _i, _i, _f, _vp],
        "launch_attention_all_heads_batch": [_vp] * 7 + [_i, _i, _i, _i, _f, _i, _i, _vp],
    }
    for name, args in sigs.items():
        getattr(lib, name).argtypes = args
        getattr(lib, name).restype = None
    return lib


@pytest.fixture(scope="module")
def eng():
    from turbo_lossless_b200 import Split12Engine
    return Split12Engine()


@pytest.fixture(scope="module")
def S():
    from oracle import step_oracle
    return step_oracle


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _st():
    return torch.cuda.current_stream().cuda_stream


def _bf16_ulps(S, a, b):
    """Largest difference of two bf16 arrays in units of the last place of the larger magnitude."""
    fa, fb = S.bf16_to_f32(a).astype(np.float64), S.bf16_to_f32(b).astype(np.float64)
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.maximum(np.abs(fa), np.abs(fb)), 1e-30))) - 7)
    return float(np.max(np.abs(fa - fb) / ulp))


def test_norms_silu_add_embed(ref, eng, S):
    rng = np.random.default_rng(1)
    n, batch, eps = 4096, 3, 1e-5
    x = rng.standard_normal((batch, n)).astype(np.float32) * 3
    res = rng.standard_normal((batch, n)).astype(np.float32)
    wgt = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    xd, wd = _cuda(x), _cuda(wgt)
    y_ref = torch.zeros((batch, n), dtype=torch.int16, device="cuda")
    y_our = torch.zeros_like(y_ref)
    ref.launch_rms_norm_bf16_batch(xd.data_ptr(), wd.data_ptr(), y_ref.data_ptr(), n, eps, batch, _st())
    eng.rms_norm_bf16(xd, wd, y_our, eps, batch)
    torch.cuda.synchronize()
    _, want = S.rms_norm_bf16(x, wgt, eps)
    assert _bf16_ulps(S, y_ref.cpu().numpy(), want) <= 1, "reference kernel vs oracle"
    assert _bf16_ulps(S, y_our.cpu().numpy(), y_ref.cpu().numpy()) <= 1, "this library vs reference kernel"
    # add + norm, with the sum written back
    x1, x2, rd = _cuda(x), _cuda(x), _cuda(res)
    ref.launch_add_rms_norm_bf16_batch(x1.data_ptr(), rd.data_ptr(), wd.data_ptr(), y_ref.data_ptr(), n, eps, batch, _st())
    eng.rms_norm_bf16(x2, wd, y_our, eps, batch, residual=rd)
    torch.cuda.synchronize()
    xs, want = S.rms_norm_bf16(x, wgt, eps, residual=res)
    assert torch.equal(x1, x2) and np.array_equal(x1.cpu().numpy(), xs)
    assert _bf16_ulps(S, y_ref.cpu().numpy(), want) <= 1
    assert _bf16_ulps(S, y_our.cpu().numpy(), y_ref.cpu().numpy()) <= 1
    # SiLU(gate) * up -> bf16, and the residual add
    nff = 14336
    gate, up = rng.standard_normal((batch, nff)).astype(np.float32) * 2, rng.standard_normal((batch, nff)).astype(np.float32)
    gd, ud = _cuda(gate), _cuda(up)
    o_ref = torch.zeros((batch, nff), dtype=torch.int16, device="cuda")
    o_our = torch.zeros_like(o_ref)
    ref.launch_silu_mul_bf16_batch(gd.data_ptr(), ud.data_ptr(), o_ref.data_ptr(), nff, batch, _st())
    eng.silu_mul_bf16(gd, ud, o_our, nff, batch)
    torch.cuda.synchronize()
    assert _bf16_ulps(S, o_ref.cpu().numpy(), S.silu_mul_bf16(gate, up)) <= 1
    assert _bf16_ulps(S, o_our.cpu().numpy(), o_ref.cpu().numpy()) <= 1
    a1, a2 = _cuda(x), _cuda(x)
    ref.launch_add_batch(a1.data_ptr(), rd.data_ptr(), n, batch, _st())
    eng.add(a2, rd, n, batch)
    torch.cuda.synchronize()
    assert torch.equal(a1, a2)
    # embedding rows, with a token outside the table
    table = S.f32_to_bf16(rng.standard_normal((500, 256)).astype(np.float32)).reshape(500, 256).view(np.int16)
    toks = np.array([0, 499, 500, -1, 17], np.int32)
    td, kd = _cuda(table), _cuda(toks)
    e_ref, e_our = torch.full((5, 256), 7.0, device="cuda"), torch.full((5, 256), 7.0, device="cuda")
    ref.launch_embed_lookup(td.data_ptr(), kd.data_ptr(), e_ref.data_ptr(), 256, 5, 500, _st())
    eng.embed_lookup(td, kd, e_our)
    torch.cuda.synchronize()
    assert torch.equal(e_ref, e_our) and np.array_equal(e_ref.cpu().numpy(), S.embed_lookup(table.view(np.uint16), toks))


@pytest.mark.parametrize("n", [1000, 32000, 128256])
def test_argmax_and_its_tie_rule(ref, eng, S, n):
    rng = np.random.default_rng(n)
    batch = 4
    logits = rng.standard_normal((batch, n)).astype(np.float32)
    for b in range(1, batch):                        # several equal maxima: the winner depends on the reduction tree
        logits[b, rng.integers(0, n, 2 + 3 * b)] = 9.0
    ld = _cuda(logits)
    r_ref = torch.full((batch,), -1, dtype=torch.int32, device="cuda")
    r_our = torch.full((batch,), -1, dtype=torch.int32, device="cuda")
    ref.launch_argmax_batch(ld.data_ptr(), r_ref.data_ptr(), n, batch, _st())
    eng.argmax(ld, r_our)
    torch.cuda.synchronize()
    assert torch.equal(r_ref, r_our)
    assert [S.argmax_engine(logits[b]) for b in range(batch)] == r_ref.cpu().tolist()
    one_ref = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    ref.launch_argmax(ld[2].data_ptr(), one_ref.data_ptr(), n, _st())
    torch.cuda.synchronize()
    assert int(one_ref[0]) == int(r_our[2])


def test_rope_store_attention(ref, eng, S):
    rng = np.random.default_rng(5)
    n_head, n_kv, hd, max_seq, theta = 32, 8, 128, 384, 10000.0
    kv_dim = n_kv * hd
    caches = {}
    for who in ("ref", "our"):
        caches[who] = (torch.zeros((max_seq, n_kv, hd), dtype=torch.int8, device="cuda"), torch.zeros((max_seq, n_kv, hd), dtype=torch.int8, device="cuda"),
                       torch.zeros((max_seq, n_kv), device="cuda"), torch.zeros((max_seq, n_kv), device="cuda"))
    for pos in (0, 1, 7, 63):
        q = rng.standard_normal(n_head * hd).astype(np.float32)
        k = rng.standard_normal(kv_dim).astype(np.float32)
        v = rng.standard_normal(kv_dim).astype(np.float32)
        out = {}
        for who in ("ref", "our"):
            qd, kd, vd = _cuda(q), _cuda(k), _cuda(v)
            kc, vc, sk, sv = caches[who]
            if who == "ref":
                ref.launch_rope_store_kv(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), kc.data_ptr(), vc.data_ptr(), sk.data_ptr(),
                                         sv.data_ptr(), hd, n_head, n_kv, pos, max_seq, theta, _st())
            else:
                eng.rope_store_kv(qd, kd, vd, kc, vc, sk, sv, hd, n_head, n_kv, pos, max_seq, theta)
            torch.cuda.synchronize()
            out[who] = (qd.cpu().numpy(), kd.cpu().numpy(), kc[pos].cpu().numpy().astype(np.int32), vc[pos].cpu().numpy().astype(np.int32),
                        sk[pos].cpu().numpy(), sv[pos].cpu().numpy())
        want_q = S.rope(q, pos, hd, theta).reshape(-1)
        want_k = S.rope(k, pos, hd, theta).reshape(-1)
        for who in ("ref", "our"):
            assert np.abs(out[who][0] - want_q).max() <= 2e-4 and np.abs(out[who][1] - want_k).max() <= 2e-4, (who, pos)
        assert np.abs(out["ref"][2] - out["our"][2]).max() <= 1            # int8 keys: one step where the rotated k differ in the last digits
        assert np.array_equal(out["ref"][3], out["our"][3])                # values are not rotated: identical
        assert np.allclose(out["ref"][4], out["our"][4], rtol=1e-4) and np.array_equal(out["ref"][5], out["our"][5])
    # attention over a random cache, single sequence and batched with per-sequence caches
    seq_len = 200
    kc = rng.integers(-127, 128, (max_seq, n_kv, hd)).astype(np.int8)
    vc = rng.integers(-127, 128, (max_seq, n_kv, hd)).astype(np.int8)
    sk = (rng.random((max_seq, n_kv)) * 0.02 + 0.001).astype(np.float32)
    sv = (rng.random((max_seq, n_kv)) * 0.02 + 0.001).astype(np.float32)
    q = rng.standard_normal(n_head * hd).astype(np.float32)
    scale = float(1.0 / np.sqrt(hd))
    dv = [_cuda(a) for a in (q, kc, vc, sk, sv)]
    o_ref = torch.zeros(n_head * hd, dtype=torch.int16, device="cuda")
    o_our = torch.zeros_like(o_ref)
    ref.launch_attention_all_heads(*[t.data_ptr() for t in dv], o_ref.data_ptr(), n_head, n_kv, hd, seq_len, max_seq, scale, _st())
    eng.attention_all_heads(*dv, o_our, n_head, n_kv, hd, seq_len, max_seq, scale)
    torch.cuda.synchronize()
    want = S.bf16_to_f32(S.attention(q, kc, vc, sk, sv, seq_len, n_head, n_kv, hd, scale)).astype(np.float64)
    for got in (o_ref, o_our):
        g = S.bf16_to_f32(got.cpu().numpy()).astype(np.float64)
        assert np.abs(g - want).max() <= 2.0 ** -7 * np.abs(want).max()
    batch = 3
    kcb = rng.integers(-127, 128, (batch, max_seq, n_kv, hd)).astype(np.int8)
    vcb = rng.integers(-127, 128, (batch, max_seq, n_kv, hd)).astype(np.int8)
    skb = (rng.random((batch, max_seq, n_kv)) * 0.02 + 0.001).astype(np.float32)
    svb = (rng.random((batch, max_seq, n_kv)) * 0.02 + 0.001).astype(np.float32)
    qb = rng.standard_normal((batch, n_head * hd)).astype(np.float32)
    pos = np.array([5, 150, 300], np.int32)
    dvb = [_cuda(a) for a in (qb, kcb, vcb, skb, svb)]
    pd = _cuda(pos)
    ob_ref = torch.zeros((batch, n_head * hd), dtype=torch.int16, device="cuda")
    ob_our = torch.zeros_like(ob_ref)
    ref.launch_attention_all_heads_batch(*[t.data_ptr() for t in dvb], ob_ref.data_ptr(), pd.data_ptr(), n_head, n_kv, hd,
                                         int(pos.max()) + 1, scale, batch, max_seq * kv_dim, _st())
    eng.attention_all_heads_batch(*dvb, ob_our, pd, n_head, n_kv, hd, int(pos.max()) + 1, scale, batch, max_seq * kv_dim)
    torch.cuda.synchronize()
    for s in range(batch):
        want = S.bf16_to_f32(S.attention(qb[s], kcb[s], vcb[s], skb[s], svb[s], int(pos[s]) + 1, n_head, n_kv, hd, scale)).astype(np.float64)
        for got in (ob_ref, ob_our):
            g = S.bf16_to_f32(got[s].cpu().numpy()).astype(np.float64)
            assert np.abs(g - want).max() <= 2.0 ** -7 * np.abs(want).max()
    assert eng.device_status() == 0


def test_batched_rope_and_store_into_one_cache(ref, eng, S):
    """launch_rope_batch and the engine's launch_store_kv_batch (every sequence into ONE cache at its position)."""
    rng = np.random.default_rng(8)
    n_head, n_kv, hd, max_seq, theta, batch = 32, 8, 128, 64, 10000.0, 4   # same theta as above: the reference caches its frequency table per head_dim only
    kv_dim = n_kv * hd
    pos = np.array([0, 3, 9, 30], np.int32)
    q = rng.standard_normal((batch, n_head * hd)).astype(np.float32)
    k = rng.standard_normal((batch, kv_dim)).astype(np.float32)
    v = rng.standard_normal((batch, kv_dim)).astype(np.float32)
    res = {}
    for who in ("ref", "our"):
        qd, kd, vd, pd = _cuda(q), _cuda(k), _cuda(v), _cuda(pos)
        kc = torch.zeros((max_seq, n_kv, hd), dtype=torch.int8, device="cuda"); vc = torch.zeros_like(kc)
        sk = torch.zeros((max_seq, n_kv), device="cuda"); sv = torch.zeros_like(sk)
        if who == "ref":
            ref.launch_rope_batch(qd.data_ptr(), kd.data_ptr(), pd.data_ptr(), hd, n_head, n_kv, n_head * hd, kv_dim, theta, batch, _st())
            ref.launch_store_kv_batch(kd.data_ptr(), vd.data_ptr(), kc.data_ptr(), vc.data_ptr(), sk.data_ptr(), sv.data_ptr(), pd.data_ptr(),
                                      kv_dim, max_seq, n_kv, hd, batch, _st())
        else:
            eng.rope_batch(qd, kd, pd, hd, n_head, n_kv, theta, batch)
            assert eng.lib.launch_store_kv_batch(kd.data_ptr(), vd.data_ptr(), kc.data_ptr(), vc.data_ptr(), sk.data_ptr(), sv.data_ptr(),
                                                 pd.data_ptr(), kv_dim, max_seq, n_kv, hd, batch, _st()) == 0
        torch.cuda.synchronize()
        res[who] = (qd.cpu().numpy(), kd.cpu().numpy(), kc.cpu().numpy().astype(np.int32), vc.cpu().numpy().astype(np.int32), sk.cpu().numpy(), sv.cpu().numpy())
    for s in range(batch):
        want_q = S.rope(q[s], int(pos[s]), hd, theta).reshape(-1)
        for who in ("ref", "our"):
            assert np.abs(res[who][0][s] - want_q).max() <= 2e-4, (who, s)
    assert np.abs(res["ref"][1] - res["our"][1]).max() <= 2e-4
    assert np.abs(res["ref"][2] - res["our"][2]).max() <= 1 and np.array_equal(res["ref"][3], res["our"][3])
    assert np.allclose(res["ref"][4], res["our"][4], rtol=1e-4) and np.array_equal(res["ref"][5], res["our"][5])
