"""The decode-step kernels around the projections (engine/kernels.hip launchers) against the numpy
restatement in oracle/step_oracle.py.

Tolerances: bf16 outputs may differ from the float64-accumulating oracle by one bf16 unit in the
last place where a value sits on a rounding boundary; rotated q/k are fp32 with
accurate sincosf (1e-5); INT8 cache entries may differ by one step where v*127/absmax sits on .5.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from turbo_lossless_b200 import Split12Engine
    return Split12Engine()


@pytest.fixture(scope="module")
def S():
    from oracle import step_oracle
    return step_oracle


def _cuda(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _bf16_close(S, got_raw, ref_raw, ulps=1):
    got, ref = S.bf16_to_f32(got_raw).astype(np.float64), S.bf16_to_f32(ref_raw).astype(np.float64)
    tol = ulps * 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 1e-30))) - 7)        # one unit in the last place of bf16
    bad = np.abs(got - ref) > tol
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ by more than {ulps} bf16 ulp; worst {np.abs(got - ref).max()}"


def test_embed_lookup_and_out_of_range_tokens(eng, S):
    import torch
    rng = np.random.default_rng(0)
    table = S.f32_to_bf16(rng.standard_normal((1000, 4096)).astype(np.float32)).reshape(1000, 4096)
    toks = np.array([0, 999, 5, -1, 1000, 123456], dtype=np.int32)
    out = torch.full((len(toks), 4096), float("nan"), device="cuda")
    eng.embed_lookup(_cuda(table), _cuda(toks), out)
    np.testing.assert_array_equal(out.cpu().numpy(), S.embed_lookup(table, toks))


@pytest.mark.parametrize("n,batch", [(4096, 1), (4096, 7), (8192, 3), (100, 2), (5000, 1)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_rms_norm_bf16(eng, S, n, batch, with_residual):
    import torch
    rng = np.random.default_rng(n + batch)
    x = (rng.standard_normal((batch, n)) * 3).astype(np.float32)
    r = rng.standard_normal((batch, n)).astype(np.float32) if with_residual else None
    w = rng.standard_normal(n).astype(np.float32)
    xd = _cuda(x)
    y = torch.zeros((batch, n), dtype=torch.int16, device="cuda")
    eng.rms_norm_bf16(xd, _cuda(w), y, 1e-5, batch, residual=_cuda(r) if with_residual else None)
    x_ref, y_ref = S.rms_norm_bf16(x, w, 1e-5, r)
    np.testing.assert_array_equal(xd.cpu().numpy(), x_ref)              # the in-place sum is exact fp32
    _bf16_close(S, y.cpu().numpy(), y_ref)


def test_silu_mul_and_add(eng, S):
    import torch
    rng = np.random.default_rng(3)
    n, batch = 14336, 3
    g = (rng.standard_normal((batch, n)) * 4).astype(np.float32)
    u = rng.standard_normal((batch, n)).astype(np.float32)
    out = torch.zeros((batch, n), dtype=torch.int16, device="cuda")
    eng.silu_mul_bf16(_cuda(g), _cuda(u), out, n, batch)
    _bf16_close(S, out.cpu().numpy(), S.silu_mul_bf16(g, u).reshape(batch, n))
    y = _cuda(g.copy())
    eng.add(y, _cuda(u), n, batch)
    np.testing.assert_array_equal(y.cpu().numpy(), g + u)


@pytest.mark.parametrize("n", [1, 255, 256, 257, 32000, 128256])
def test_argmax_matches_engine_tie_rule(eng, S, n):
    import torch
    rng = np.random.default_rng(n)
    rows = []
    rows.append(rng.standard_normal(n).astype(np.float32))
    tie = rng.integers(0, 4, n).astype(np.float32)                      # many equal maxima
    rows.append(tie)
    one = np.full(n, -5.0, dtype=np.float32); one[n - 1] = 7.0
    rows.append(one)
    if n > 300:
        t2 = np.zeros(n, dtype=np.float32); t2[6] = 1.0; t2[261] = 1.0   # thread 6 beats thread 5 (index 261) in the engine's reduction tree
        rows.append(t2)
    logits = np.stack(rows)
    res = torch.full((len(rows),), -1, dtype=torch.int32, device="cuda")
    eng.argmax(_cuda(logits), res)
    want = [S.argmax_engine(r) for r in rows]
    assert res.cpu().numpy().tolist() == want
    for r, w in zip(rows, want):
        assert r[w] == r.max()


@pytest.mark.parametrize("n_head,n_head_kv,head_dim", [(32, 8, 128), (64, 8, 128), (8, 8, 64), (6, 2, 96)])
def test_rope_store_kv_b1(eng, S, n_head, n_head_kv, head_dim):
    import torch
    rng = np.random.default_rng(n_head * head_dim)
    max_seq, theta = 64, 10000.0
    kv_dim = n_head_kv * head_dim
    kc = torch.zeros((max_seq, n_head_kv, head_dim), dtype=torch.int8, device="cuda")
    vc = torch.zeros_like(kc)
    sk = torch.zeros((max_seq, n_head_kv), device="cuda")
    sv = torch.zeros_like(sk)
    for pos in (0, 1, 37, 63):
        q = rng.standard_normal(n_head * head_dim).astype(np.float32)
        k = rng.standard_normal(kv_dim).astype(np.float32)
        v = (rng.standard_normal(kv_dim) * 2).astype(np.float32)
        if pos == 1:
            v[:head_dim] = 0.0                                          # an all-zero head: scale 0, values 0
        qd, kd, vd = _cuda(q), _cuda(k), _cuda(v)
        eng.rope_store_kv(qd, kd, vd, kc, vc, sk, sv, head_dim, n_head, n_head_kv, pos, max_seq, theta)
        q_ref, k_ref = S.rope(q, pos, head_dim, theta), S.rope(k, pos, head_dim, theta)
        np.testing.assert_allclose(qd.cpu().numpy().reshape(-1, head_dim), q_ref, rtol=0, atol=2e-5)
        k_got = kd.cpu().numpy().reshape(-1, head_dim)
        np.testing.assert_allclose(k_got, k_ref, rtol=0, atol=2e-5)
        for h in range(n_head_kv):
            for cache, scales, src in ((kc, sk, k_got[h]), (vc, sv, v[h * head_dim:(h + 1) * head_dim])):
                qv, sc = S.quantize_head(src)                           # from the kernel's own rotated k: exact
                np.testing.assert_array_equal(cache[pos, h].cpu().numpy(), qv)
                assert scales[pos, h].item() == sc


@pytest.mark.parametrize("seq_len", [1, 2, 129, 384, 1500])
def test_attention_b1(eng, S, seq_len):
    import torch
    n_head, n_head_kv, hd, max_seq = 32, 8, 128, 2048
    rng = np.random.default_rng(seq_len)
    q = rng.standard_normal(n_head * hd).astype(np.float32)
    kc = rng.integers(-127, 128, (max_seq, n_head_kv, hd)).astype(np.int8)
    vc = rng.integers(-127, 128, (max_seq, n_head_kv, hd)).astype(np.int8)
    sk = (rng.random((max_seq, n_head_kv)) * 0.02 + 0.001).astype(np.float32)
    sv = (rng.random((max_seq, n_head_kv)) * 0.02 + 0.001).astype(np.float32)
    out = torch.zeros(n_head * hd, dtype=torch.int16, device="cuda")
    scale = 1.0 / np.sqrt(hd)
    eng.attention_all_heads(_cuda(q), _cuda(kc), _cuda(vc), _cuda(sk), _cuda(sv), out, n_head, n_head_kv, hd, seq_len,
                            max_seq, float(scale))
    ref = S.attention(q, kc, vc, sk, sv, seq_len, n_head, n_head_kv, hd, scale)
    got = S.bf16_to_f32(out.cpu().numpy()).astype(np.float64)
    want = S.bf16_to_f32(ref).astype(np.float64)
    assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()   # bf16 output of an fp32 weighted sum


def test_batched_rope_store_attention_per_sequence_caches(eng, S):
    """launch_rope_batch + s12_store_kv_batch + launch_attention_all_heads_batch with a cache per sequence."""
    import torch
    n_head, n_head_kv, hd, max_seq, B, theta = 16, 4, 128, 96, 5, 500000.0
    kv_dim = n_head_kv * hd
    kv_stride = max_seq * kv_dim
    rng = np.random.default_rng(11)
    kc = torch.zeros((B, max_seq, n_head_kv, hd), dtype=torch.int8, device="cuda")
    vc = torch.zeros_like(kc)
    sk = torch.zeros((B, max_seq, n_head_kv), device="cuda")
    sv = torch.zeros_like(sk)
    ref_k = np.zeros((B, max_seq, n_head_kv, hd), dtype=np.int8); ref_v = np.zeros_like(ref_k)
    ref_sk = np.zeros((B, max_seq, n_head_kv), dtype=np.float32); ref_sv = np.zeros_like(ref_sk)
    lens = [3, 17, 1, 40, 25]
    q_last = None
    for step in range(max(lens)):
        active = [s for s in range(B) if step < lens[s]]
        pos = np.array([step if s in active else lens[s] - 1 for s in range(B)], dtype=np.int32)   # idle ones rewrite their last slot
        q = rng.standard_normal((B, n_head * hd)).astype(np.float32)
        k = rng.standard_normal((B, kv_dim)).astype(np.float32)
        v = rng.standard_normal((B, kv_dim)).astype(np.float32)
        qd, kd = _cuda(q), _cuda(k)
        eng.rope_batch(qd, kd, _cuda(pos), hd, n_head, n_head_kv, theta, B)
        eng.store_kv_batch(kd, _cuda(v), kc, vc, sk, sv, _cuda(pos), n_head_kv, hd, B, kv_stride=kv_stride)
        k_rot = kd.cpu().numpy()
        for s in range(B):
            np.testing.assert_allclose(k_rot[s].reshape(-1, hd), S.rope(k[s], int(pos[s]), hd, theta), rtol=0, atol=2e-5)
            for h in range(n_head_kv):
                ref_k[s, pos[s], h], ref_sk[s, pos[s], h] = S.quantize_head(k_rot[s, h * hd:(h + 1) * hd])
                ref_v[s, pos[s], h], ref_sv[s, pos[s], h] = S.quantize_head(v[s, h * hd:(h + 1) * hd])
        q_last, pos_last = qd.cpu().numpy(), pos
    np.testing.assert_array_equal(kc.cpu().numpy(), ref_k)
    np.testing.assert_array_equal(vc.cpu().numpy(), ref_v)
    np.testing.assert_array_equal(sk.cpu().numpy(), ref_sk)
    out = torch.zeros((B, n_head * hd), dtype=torch.int16, device="cuda")
    scale = float(1.0 / np.sqrt(hd))
    eng.attention_all_heads_batch(_cuda(q_last), kc, vc, sk, sv, out, _cuda(pos_last), n_head, n_head_kv, hd,
                                  int(pos_last.max()) + 1, scale, B, kv_stride)
    got = S.bf16_to_f32(out.cpu().numpy()).astype(np.float64)
    for s in range(B):
        ref = S.attention(q_last[s], ref_k[s], ref_v[s], ref_sk[s], ref_sv[s], int(pos_last[s]) + 1, n_head, n_head_kv, hd, scale)
        want = S.bf16_to_f32(ref).astype(np.float64)
        assert np.abs(got[s] - want).max() <= 2.0 ** -7 * np.abs(want).max()


def test_flash_attention_names_forward_to_the_same_kernels(eng, S):
    """The engine calls launch_flash_attention[_batch] from position 1024 on (engine/inference.cpp:285,432):
    same arguments, same results as launch_attention_all_heads[_batch], checked against the oracle at 1500
    positions, and at 9000 positions for 80 (sequence, kv head) pairs with four query heads each: one slice's
    scores no longer fit a CTA's shared memory, so the positions are cut in two although the GPU is already full."""
    import torch
    n_head, n_head_kv, hd, max_seq, seq_len = 32, 8, 128, 2048, 1500
    rng = np.random.default_rng(77)
    q = rng.standard_normal(n_head * hd).astype(np.float32)
    kc = rng.integers(-127, 128, (max_seq, n_head_kv, hd)).astype(np.int8)
    vc = rng.integers(-127, 128, (max_seq, n_head_kv, hd)).astype(np.int8)
    sk = (rng.random((max_seq, n_head_kv)) * 0.02 + 0.001).astype(np.float32)
    sv = (rng.random((max_seq, n_head_kv)) * 0.02 + 0.001).astype(np.float32)
    scale = float(1.0 / np.sqrt(hd))
    qd, kd, vd, skd, svd = _cuda(q), _cuda(kc), _cuda(vc), _cuda(sk), _cuda(sv)
    out = torch.zeros(n_head * hd, dtype=torch.int16, device="cuda")
    out2 = torch.zeros_like(out)
    eng.attention_all_heads(qd, kd, vd, skd, svd, out, n_head, n_head_kv, hd, seq_len, max_seq, scale)
    st = torch.cuda.current_stream().cuda_stream
    rc = eng.lib.launch_flash_attention(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), skd.data_ptr(), svd.data_ptr(),
                                        out2.data_ptr(), n_head, n_head_kv, hd, seq_len, max_seq, scale, st)
    assert rc == 0
    assert torch.equal(out, out2)
    want = S.bf16_to_f32(S.attention(q, kc, vc, sk, sv, seq_len, n_head, n_head_kv, hd, scale)).astype(np.float64)
    got = S.bf16_to_f32(out2.cpu().numpy()).astype(np.float64)
    assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()

    # batched name, long context, many sequences
    batch, n_head, n_head_kv, long_seq = 20, 16, 4, 9000
    kv_stride = long_seq * n_head_kv * hd
    qb = rng.standard_normal((batch, n_head * hd)).astype(np.float32)
    kcb = rng.integers(-127, 128, (batch, long_seq, n_head_kv, hd)).astype(np.int8)
    vcb = rng.integers(-127, 128, (batch, long_seq, n_head_kv, hd)).astype(np.int8)
    skb = (rng.random((batch, long_seq, n_head_kv)) * 0.02 + 0.001).astype(np.float32)
    svb = (rng.random((batch, long_seq, n_head_kv)) * 0.02 + 0.001).astype(np.float32)
    pos = rng.integers(7000, long_seq, batch).astype(np.int32)
    pos[0] = long_seq - 1
    outb = torch.zeros((batch, n_head * hd), dtype=torch.int16, device="cuda")
    dv = [_cuda(a) for a in (qb, kcb, vcb, skb, svb, pos)]          # kept alive until the kernel has run
    rc = eng.lib.launch_flash_attention_batch(dv[0].data_ptr(), dv[1].data_ptr(), dv[2].data_ptr(), dv[3].data_ptr(),
                                              dv[4].data_ptr(), outb.data_ptr(), dv[5].data_ptr(), n_head, n_head_kv, hd,
                                              long_seq, scale, batch, kv_stride, st)
    assert rc == 0, eng.lib.s12_last_error()
    torch.cuda.synchronize()
    for s in (0, 7, batch - 1):
        want = S.bf16_to_f32(S.attention(qb[s], kcb[s], vcb[s], skb[s], svb[s], int(pos[s]) + 1, n_head, n_head_kv, hd,
                                         scale)).astype(np.float64)
        got = S.bf16_to_f32(outb[s].cpu().numpy()).astype(np.float64)
        assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()
    assert eng.device_status() == 0
