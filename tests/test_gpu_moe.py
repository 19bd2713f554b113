"""Top-2 mixture-of-experts block (route, gather, expert projections, combine) against the numpy statement in
oracle/step_oracle.py.  Routing, lists and slots are integer work: exact.  Outputs: activations are rounded to
bf16 between the projections, so 2 % of the largest magnitude, as in the decoder test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def route_on_device(logits):
    import torch
    from turbo_lossless_b200 import capi
    from turbo_lossless_b200.capi import check
    lib = capi.load()
    T, E = logits.shape
    d = torch.from_numpy(logits).cuda()
    sel = torch.zeros(T, 2, dtype=torch.int32).cuda(); wt = torch.zeros(T, 2).cuda(); slot = torch.full((T, 2), -1, dtype=torch.int32).cuda()
    lists = torch.full((E, T), -1, dtype=torch.int32).cuda(); counts = torch.zeros(E, dtype=torch.int32).cuda()
    check(lib.s12_moe_route_async(d.data_ptr(), T, E, sel.data_ptr(), wt.data_ptr(), slot.data_ptr(), lists.data_ptr(),
                                  counts.data_ptr(), None), "route")
    torch.cuda.synchronize()
    return [a.cpu().numpy() for a in (sel, wt, slot, lists, counts)]


@pytest.mark.parametrize("T,E", [(64, 8), (1, 8), (7, 2), (300, 32), (5, 1), (40, 3)])
def test_routing_lists_and_slots(T, E):
    from oracle import step_oracle as S
    rng = np.random.default_rng(T * 100 + E)
    logits = rng.uniform(-1, 1, (T, E)).astype(np.float32)
    logits[0, :] = 0.25                                            # a full tie: experts 0 and 1
    if T > 3 and E > 2:
        logits[3, -1] = logits[3, 0] = 5.0                         # a two-way tie at the top
    sel, wt, slot, lists, counts = route_on_device(logits)
    rsel, rwt = S.moe_route(logits)
    assert np.array_equal(sel, rsel)
    assert np.abs(wt - rwt).max() < 1e-6 and np.allclose(wt.sum(1), 1.0, atol=1e-6)
    for e in range(E):
        want = [t for t in range(T) if (rsel[t, 0] == e) or (rsel[t, 1] == e and rwt[t, 1] != 0)]
        assert counts[e] == len(want) and list(lists[e, :len(want)]) == want
        for i, t in enumerate(want):
            k = 0 if rsel[t, 0] == e else 1
            assert slot[t, k] == i
    assert counts.sum() == (2 * T if E > 1 else T)


@pytest.mark.parametrize("T,capacity", [(64, None), (16, None), (3, None), (1, None), (20, 40)])
def test_moe_block_matches_the_oracle(O, T, capacity):
    import torch
    from oracle import step_oracle as S
    from turbo_lossless_b200 import CompressedWeight
    from turbo_lossless_b200.moe import MoEFeedForward
    E, H, F = 8, 256, 512
    rng = np.random.default_rng(T)
    raw, experts = [], []
    for e in range(E):
        ws = [O.synth_weights(F, H, 10 * e, std=0.06, outlier_frac=2.5e-3), O.synth_weights(F, H, 10 * e + 1, std=0.06, outlier_frac=2.5e-3),
              O.synth_weights(H, F, 10 * e + 2, std=0.06, outlier_frac=2.5e-3)]
        raw.append(tuple(ws))
        experts.append({n: CompressedWeight.from_packed(O.pack(w)) for n, w in zip(("w_gate", "w_up", "w_down"), ws)})
    x = S.f32_to_bf16(rng.standard_normal((T, H)).astype(np.float32)).reshape(T, H)
    logits = rng.uniform(-1, 1, (T, E)).astype(np.float32)
    moe = MoEFeedForward(experts, T, capacity)
    out = torch.full((T, H), 3.0, device="cuda")
    moe.forward(torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda(), out)
    torch.cuda.synchronize()
    assert moe.eng.device_status() == 0
    want = S.moe_ffn(x, logits, raw, lambda W, xr: O.gemm_exact(W, xr.view(np.uint16)))
    got = out.cpu().numpy()
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    # accumulate adds to what is there; a second call gives the same bits (deterministic)
    out2 = torch.full((T, H), 3.0, device="cuda")
    moe.forward(torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda(), out2, accumulate=True)
    torch.cuda.synchronize()
    assert np.abs(out2.cpu().numpy() - 3.0 - got).max() <= 1e-5 * max(1.0, np.abs(got).max())
    out3 = torch.empty((T, H), device="cuda")
    moe.forward(torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda(), out3)
    torch.cuda.synchronize()
    assert np.array_equal(out3.cpu().numpy(), got)


def test_bad_arguments_are_refused():
    import torch
    from turbo_lossless_b200 import capi
    lib = capi.load()
    z = torch.zeros(64, dtype=torch.int32).cuda()
    p = z.data_ptr()
    assert lib.s12_moe_route_async(p, 4, 33, p, p, p, p, p, None) < 0      # more experts than a warp has lanes
    assert lib.s12_moe_route_async(None, 4, 8, p, p, p, p, p, None) < 0
    assert lib.s12_moe_gather_async(p, 0, 4, 8, 4, p, p, p, None) < 0
    assert lib.s12_moe_combine_async(p, 8, 4, 0, p, p, p, p, 0, None) < 0


@pytest.mark.parametrize("B", [17, 64, 8])
def test_grouped_gemm_reads_each_tensors_own_rows(O, B):
    """s12_gemm_grouped_async: six tensors of different heights, each with its own block of B activation rows."""
    import torch
    from oracle import step_oracle as S
    from turbo_lossless_b200 import CompressedWeight, Split12Engine
    K, Ms = 512, [128, 300, 64, 256, 130, 512]
    rng = np.random.default_rng(B)
    raw = [O.synth_weights(M, K, 40 + i, std=0.06, outlier_frac=2e-3) for i, M in enumerate(Ms)]
    ws = [CompressedWeight.from_packed(O.pack(w)) for w in raw]
    row0 = [0, B, 2 * B, 2 * B, 5 * B, 3 * B]                        # two tensors share a block, one block is unused
    x = S.f32_to_bf16(rng.standard_normal((6 * B, K)).astype(np.float32)).reshape(6 * B, K)
    outs = [torch.full((B, M), np.nan, device="cuda") for M in Ms]
    eng = Split12Engine()
    eng.gemm_grouped(ws, torch.from_numpy(x).cuda(), row0, outs, K, B)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    for w, r, o in zip(raw, row0, outs):
        want = O.gemm_exact(w, x[r:r + B].view(np.uint16))
        assert np.abs(o.cpu().numpy() - want).max() <= 1e-3 * np.abs(want).max()
