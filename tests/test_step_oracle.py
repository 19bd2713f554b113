"""CPU checks of the numpy restatement of the engine's decode-step kernels (oracle/step_oracle.py):
properties that follow from the kernels' definitions in engine/kernels.hip."""
import numpy as np

from oracle import step_oracle as S


def test_bf16_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 0.0, 3.0e38], dtype=np.float32)
    raw = S.f32_to_bf16(x)
    back = S.bf16_to_f32(raw)
    assert back[0] == 1.0 and back[3] == -2.5 and back[4] == 0.0
    assert back[1] == 1.0                 # 1 + 2^-8 is a tie between 1 and 1 + 2^-7: even mantissa wins
    assert back[2] == np.float32(1.015625)   # 1 + 3*2^-8 ties up to 1 + 2^-6
    assert np.all(np.abs(back[:5] - x[:5]) <= np.abs(x[:5]) * 2.0 ** -8)


def test_argmax_tie_rule_is_the_reduction_tree():
    n = 1000
    t = np.zeros(n, dtype=np.float32)
    t[6] = t[261] = 1.0                  # thread 6 (i = 6) against thread 5 (i = 261)
    assert S.argmax_engine(t) == 6       # slot 2 feeds slot 0 at stride 2; slot 1 loses the last tie to slot 0
    t[:] = 0.0
    assert S.argmax_engine(t) == 0
    t[700] = 5.0
    assert S.argmax_engine(t) == 700
    t[700 - 256] = 5.0                   # same thread, earlier index
    assert S.argmax_engine(t) == 700 - 256


def test_quantize_head_and_rope_properties():
    rng = np.random.default_rng(0)
    v = rng.standard_normal(128).astype(np.float32)
    q, sc = S.quantize_head(v)
    assert q.dtype == np.int8 and np.abs(q).max() == 127
    assert np.abs(q.astype(np.float32) * sc - v).max() <= sc * 0.5 * (1 + 1e-6)
    qz, scz = S.quantize_head(np.zeros(64, dtype=np.float32))
    assert scz == 0 and not qz.any()
    x = rng.standard_normal((4, 128)).astype(np.float32)
    r = S.rope(x, 37, 128, 10000.0)
    np.testing.assert_allclose((r ** 2).sum(axis=1), (x ** 2).sum(axis=1), rtol=1e-5)   # rotations keep the norm
    np.testing.assert_array_equal(S.rope(x, 0, 128, 10000.0), x)


def test_rms_norm_and_attention_small():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, 64)).astype(np.float32)
    w = np.ones(64, dtype=np.float32)
    xs, y = S.rms_norm_bf16(x, w, 0.0)
    yf = S.bf16_to_f32(y).astype(np.float64)
    np.testing.assert_allclose((yf ** 2).mean(axis=1), 1.0, rtol=2e-2)
    # one cached position: the output is that position's value row
    kc = rng.integers(-127, 128, (4, 2, 8)).astype(np.int8)
    vc = rng.integers(-127, 128, (4, 2, 8)).astype(np.int8)
    sk = np.full((4, 2), 0.01, dtype=np.float32); sv = np.full((4, 2), 0.02, dtype=np.float32)
    q = rng.standard_normal(4 * 8).astype(np.float32)
    out = S.bf16_to_f32(S.attention(q, kc, vc, sk, sv, 1, 4, 2, 8, 8 ** -0.5)).reshape(4, 8)
    for h in range(4):
        np.testing.assert_allclose(out[h], vc[0, h // 2].astype(np.float32) * 0.02, rtol=2 ** -8)


def test_moe_route_and_block_statement():
    """Top-2 routing: ties go to the lower expert, the two weights are the softmax over the two logits; the block
    is the weighted sum of the chosen experts' SwiGLU outputs."""
    from oracle import step_oracle as S
    logits = np.array([[0.0, 2.0, 2.0, -1.0], [1.0, 0.0, 0.0, 0.0], [0.5, 0.5, 0.5, 0.5]], np.float32)
    sel, wt = S.moe_route(logits)
    assert sel.tolist() == [[1, 2], [0, 1], [0, 1]]
    assert np.allclose(wt[0], [0.5, 0.5]) and np.allclose(wt[1], [np.e / (1 + np.e), 1 / (1 + np.e)])
    sel1, wt1 = S.moe_route(np.zeros((2, 1), np.float32))
    assert sel1.tolist() == [[0, 0], [0, 0]] and wt1.tolist() == [[1.0, 0.0], [1.0, 0.0]]
    rng = np.random.default_rng(0)
    H, F, E = 8, 16, 4
    experts = [tuple(rng.standard_normal(s) for s in ((F, H), (F, H), (H, F))) for _ in range(E)]
    x = S.f32_to_bf16(rng.standard_normal((3, H)).astype(np.float32)).reshape(3, H)
    mm = lambda W, xr: S.bf16_to_f32(xr).astype(np.float64) @ W.T  # noqa: E731
    out = S.moe_ffn(x, logits, experts, mm)
    t = 1
    want = np.zeros(H)
    for k in range(2):
        g, u, d = experts[sel[t, k]]
        h = S.silu_mul_bf16((mm(g, x[t:t + 1])).astype(np.float32), (mm(u, x[t:t + 1])).astype(np.float32)).reshape(1, -1)
        want += wt[t, k] * mm(d, h)[0]
    assert np.allclose(out[t], want, rtol=1e-6)
