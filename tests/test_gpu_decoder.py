"""A whole decode step (turbo_lossless_b200.decoder.Decoder) against a numpy forward pass built from the
oracle's pieces: split12 unpack + float64 matmul for the projections, oracle/step_oracle.py for the rest.

Tolerance: activations are rounded to bf16 between operations and KV entries to int8, so the two
passes may round a value differently now and then; logits agree to 2 % of their largest magnitude and
the greedy token agrees whenever the oracle's top two logits are further apart than that.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class NumpyDecoder:
    def __init__(self, O, S, cfg, w, embd, norms, batch):
        self.O, self.S, self.cfg, self.w, self.embd, self.norms, self.B = O, S, cfg, w, embd, norms, batch
        hd = cfg.head_dim
        self.kv_k = np.zeros((cfg.n_layer, batch, cfg.max_seq, cfg.n_head_kv, hd), dtype=np.int8)
        self.kv_v = np.zeros_like(self.kv_k)
        self.sc_k = np.zeros((cfg.n_layer, batch, cfg.max_seq, cfg.n_head_kv), dtype=np.float32)
        self.sc_v = np.zeros_like(self.sc_k)

    def proj(self, name, li, x_bf16):
        W = self.w[(name, li)]
        return self.O.gemm_exact(W, x_bf16.view(np.uint16))

    def forward(self, tokens, positions):
        S, c = self.S, self.cfg
        hd = c.head_dim
        cur = S.embed_lookup(self.embd, tokens)
        res = None
        _, a = S.rms_norm_bf16(cur, self.norms["attn_norm.0"], c.rms_norm_eps)
        for li in range(c.n_layer):
            q, k, v = (self.proj(nm, li, a).astype(np.float32) for nm in ("wq", "wk", "wv"))
            attn = np.zeros((self.B, c.n_embd), dtype=np.int16)
            for s in range(self.B):
                p = int(positions[s])
                qr = S.rope(q[s], p, hd, c.rope_theta).reshape(-1)
                kr = S.rope(k[s], p, hd, c.rope_theta)
                for h in range(c.n_head_kv):
                    self.kv_k[li, s, p, h], self.sc_k[li, s, p, h] = S.quantize_head(kr[h])
                    self.kv_v[li, s, p, h], self.sc_v[li, s, p, h] = S.quantize_head(v[s, h * hd:(h + 1) * hd])
                attn[s] = S.attention(qr, self.kv_k[li, s], self.kv_v[li, s], self.sc_k[li, s], self.sc_v[li, s], p + 1,
                                      c.n_head, c.n_head_kv, hd, 1.0 / np.sqrt(hd))
            o = self.proj("wo", li, attn).astype(np.float32)
            res, a = S.rms_norm_bf16(o, self.norms[f"ffn_norm.{li}"], c.rms_norm_eps, residual=cur)
            g, u = self.proj("w_gate", li, a).astype(np.float32), self.proj("w_up", li, a).astype(np.float32)
            b = S.silu_mul_bf16(g, u).reshape(self.B, -1)
            d = self.proj("w_down", li, b).astype(np.float32)
            nxt = self.norms[f"attn_norm.{li + 1}"] if li + 1 < c.n_layer else self.norms["output_norm"]
            cur, a = S.rms_norm_bf16(d, nxt, c.rms_norm_eps, residual=res)
        return self.proj("lm_head", 0, a).astype(np.float32)


@pytest.mark.parametrize("batch", [1, 3, 20])
def test_decode_steps_match_numpy_forward(batch):
    import torch
    from oracle import oracle as O, step_oracle as S
    from turbo_lossless_b200 import CompressedWeight, Decoder, DecoderConfig
    cfg = DecoderConfig(n_embd=256, n_head=4, n_head_kv=2, n_ff=512, n_vocab=1000, n_layer=2, max_seq=32, rope_theta=10000.0)
    rng = np.random.default_rng(5)
    shapes = {"wq": (256, 256), "wk": (128, 256), "wv": (128, 256), "wo": (256, 256), "w_gate": (512, 256),
              "w_up": (512, 256), "w_down": (256, 512)}
    w, layers = {}, []
    for li in range(cfg.n_layer):
        L = {}
        for i, (nm, (M, K)) in enumerate(shapes.items()):
            w[(nm, li)] = O.synth_weights(M, K, 100 * li + i, std=0.06, outlier_frac=1e-3)
            L[nm] = CompressedWeight.from_packed(O.pack(w[(nm, li)]))
        layers.append(L)
    w[("lm_head", 0)] = O.synth_weights(cfg.n_vocab, 256, 999, std=0.06, outlier_frac=1e-3)
    lm_head = CompressedWeight.from_packed(O.pack(w[("lm_head", 0)]))
    embd = S.f32_to_bf16(rng.standard_normal((cfg.n_vocab, 256)).astype(np.float32)).reshape(cfg.n_vocab, 256)
    names = [f"attn_norm.{i}" for i in range(cfg.n_layer)] + [f"ffn_norm.{i}" for i in range(cfg.n_layer)] + ["output_norm"]
    norms = {nm: (1.0 + 0.1 * rng.standard_normal(256)).astype(np.float32) for nm in names}
    dec = Decoder(cfg, layers, lm_head, torch.from_numpy(embd).cuda(), {k: torch.from_numpy(v).cuda() for k, v in norms.items()},
                  batch=batch)
    ref = NumpyDecoder(O, S, cfg, w, embd, norms, batch)
    toks = rng.integers(0, cfg.n_vocab, batch).astype(np.int32)
    pos = np.arange(batch, dtype=np.int32) % 3                       # sequences at different positions
    agree = total = 0
    for step in range(5):
        dec.tokens.copy_(torch.from_numpy(toks)); dec.positions.copy_(torch.from_numpy(pos))
        dec.forward()
        torch.cuda.synchronize()
        assert dec.eng.device_status() == 0
        got = dec.logits.cpu().numpy()
        want = ref.forward(toks, pos)
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max(), f"step {step}"
        nxt = dec.next_tokens.cpu().numpy()
        for s in range(batch):
            top2 = np.sort(want[s])[-2:]
            if top2[1] - top2[0] > 4e-2 * np.abs(want).max():
                total += 1
                agree += int(nxt[s] == int(np.argmax(want[s])))
            assert got[s, nxt[s]] == got[s].max()
        toks = np.argmax(want, axis=1).astype(np.int32)             # both continue from the oracle's choice
        pos = pos + 1
    assert agree == total
