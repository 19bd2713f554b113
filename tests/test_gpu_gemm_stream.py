"""The streaming small-batch kernel (gemm_stream.cu) behind s12_gemv_batched_async and s12_gemm_async, against the
oracle.  By default it takes 2 <= B <= 8 on tensors of 64 row tiles or more and 9 <= B <= 16 on 24 M weights or more; S12_GSTREAM=2 forces it on smaller
shapes, S12_GSTREAM_MAXB=32 on 17..32 sequences (its four-column-tile form), S12_GSTREAM=0 turns it off (the kernels
that serve those cases otherwise are the second opinion)."""
import numpy as np
import pytest
import torch

from gpu_util import REL_TOL, assert_close, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from turbo_lossless_b200 import Split12Engine
    return Split12Engine()


def _cw(p, **kw):
    from turbo_lossless_b200 import CompressedWeight
    return CompressedWeight.from_packed(p, **kw)


def _run(eng, cw, xd, M, K, B, act_stride=None, out_stride=None, exact=True):
    act_stride, out_stride = act_stride or K, out_stride or M
    out = torch.full((B, out_stride), float("nan"), device="cuda")
    if B <= 16:
        eng.gemv_batched(cw, xd, out, act_stride, out_stride, B, exact=exact)
    else:
        eng.gemm(cw, xd, out, act_stride, out_stride, B, exact=exact)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("B", [2, 3, 8, 9, 16, 17, 24, 32])
@pytest.mark.parametrize("M,K", [(128, 256), (300, 512), (130, 1056), (1000, 4128), (4096, 4096), (700, 14336)])
def test_exact_against_the_oracle(eng, O, monkeypatch, M, K, B):
    """Ragged row counts, K that is not a multiple of the 256-column stage, escapes in 0.2 % of the weights,
    padded activation and output rows.  Two runs are bit-identical."""
    monkeypatch.setenv("S12_GSTREAM", "2")
    monkeypatch.setenv("S12_GSTREAM_MAXB", "32")
    w = O.synth_weights(M, K, M + K + B, outlier_frac=2e-3)
    p = O.pack(w)
    x = O.synth_acts(B, K, B)
    act_stride, out_stride = K + 64, M + 8
    xd = torch.zeros((B, act_stride), dtype=torch.int16, device="cuda")
    xd[:, :K] = dev(x)
    cw = _cw(p)
    out = _run(eng, cw, xd, M, K, B, act_stride, out_stride)
    assert eng.device_status() == 0
    assert_close(out[:, :M], O.gemm_exact(w, x), what="streaming kernel")
    assert torch.isnan(out[:, M:]).all()
    again = _run(eng, cw, xd, M, K, B, act_stride, out_stride)
    assert torch.equal(out[:, :M], again[:, :M])
    # the kernels that served this range before give the same numbers within the tolerance
    monkeypatch.setenv("S12_GSTREAM", "0")
    old = _run(eng, cw, xd, M, K, B, act_stride, out_stride)
    ref = O.gemm_exact(w, x)
    assert np.abs(old[:, :M].cpu().numpy() - out[:, :M].cpu().numpy()).max() <= 2 * REL_TOL * np.abs(ref).max()


@pytest.mark.parametrize("knobs", [{"S12_GSTREAM_MAXGRID": "1"},                               # one CTA walks every tile
                                   {"S12_GSTREAM_WHOLE": "0", "S12_GSTREAM_MAXGRID": "7", "S12_GSTREAM_MINIT": "1"},   # tiles cut between two CTAs
                                   {"S12_GSTREAM_WHOLE": "0", "S12_GSTREAM_MINIT": "3"},       # a tile spans five or six CTAs
                                   {"S12_GSTREAM_WHOLE": "0", "S12_GSTREAM_MINIT": "1"},       # every CTA holds one or two stages
                                   {"S12_GSTREAM_WHOLE": "1"},                                 # whole tiles, one or more per CTA
                                   {"S12_GSTREAM_WHOLE": "1", "S12_GSTREAM_GRID": "3"},
                                   {"S12_GSTREAM_STAGES": "2"}, {"S12_GSTREAM_STAGES": "4"}])
@pytest.mark.parametrize("M,K,B", [(256, 4096, 4), (900, 2048, 12), (1500, 1024, 32)])
def test_every_cut_of_the_iteration_space(eng, O, monkeypatch, knobs, M, K, B):
    """Both schedules: stream-K ranges (owners that wait for one or for many contributors, CTAs whose whole range
    lies inside one tile) and whole tiles; ring depths.  The result does not depend on the cut beyond the order of fp32 additions, and
    two runs of one cut are bit-identical."""
    monkeypatch.setenv("S12_GSTREAM", "2")
    monkeypatch.setenv("S12_GSTREAM_MAXB", "32")
    for k, v in knobs.items():
        monkeypatch.setenv(k, v)
    w = O.synth_weights(M, K, M + B, outlier_frac=2e-3)
    p = O.pack(w)
    x = O.synth_acts(B, K, 5)
    cw, xd = _cw(p), dev(x)
    outs = [_run(eng, cw, xd, M, K, B) for _ in range(2)]
    assert eng.device_status() == 0
    assert_close(outs[0], O.gemm_exact(w, x), what=str(knobs))
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("B", [4, 16, 32])
@pytest.mark.parametrize("whole", ["0", "1"])
def test_multi_tensor_launch_qkv(eng, O, monkeypatch, B, whole):
    """q/k/v-like tensors (own base_exp, own row counts, one ragged, one without escapes) as one launch: their row
    tiles form one schedule."""
    monkeypatch.setenv("S12_GSTREAM", "2")
    monkeypatch.setenv("S12_GSTREAM_MAXB", "32")
    monkeypatch.setenv("S12_GSTREAM_WHOLE", whole)
    monkeypatch.setenv("S12_GSTREAM_MINIT", "3")
    K = 1024
    specs = [(512, 0.02, 1e-3), (130, 0.05, 5e-3), (128, 0.01, 0.0)]
    ws, packs = [], []
    for i, (M, std, frac) in enumerate(specs):
        w = O.synth_weights(M, K, 200 + i, std=std, outlier_frac=frac)
        ws.append(w); packs.append(O.pack(w))
    x = O.synth_acts(B, K, 9)
    outs = [torch.full((B, p.M + 4), float("nan"), device="cuda") for p in packs]
    eng.gemm_multi([_cw(p) for p in packs], dev(x), outs, K, B)
    torch.cuda.synchronize()
    for w, p, o in zip(ws, packs, outs):
        assert_close(o[:, :p.M], O.gemm_exact(w, x), what=f"M={p.M}")
        assert torch.isnan(o[:, p.M:]).all()
    assert eng.device_status() == 0


def _tiny_exponent_weights(M, K, seed, escapes):
    rng = np.random.default_rng(seed)
    w = ((rng.integers(0, 2, (M, K)) << 15) | (rng.integers(1, 15, (M, K)) << 7) | rng.integers(0, 128, (M, K))).astype(np.uint16)
    w[rng.random((M, K)) < 0.02] = 0
    if escapes:
        mask = rng.random((M, K)) < 2e-3
        w[mask] = ((rng.integers(15, 19, (M, K)) << 7) | rng.integers(0, 128, (M, K))).astype(np.uint16)[mask]
    return w


@pytest.mark.parametrize("B", [4, 16, 24])
@pytest.mark.parametrize("escapes", [False, True])
def test_window_starting_at_exponent_zero(eng, O, monkeypatch, B, escapes):
    """base_exp = -1 (split12_pack.c:29-35): exact with the CSR list; without it escapes keep the reference's bits
    (exponent field 0xFF: infinities and NaNs in their rows)."""
    monkeypatch.setenv("S12_GSTREAM", "2")
    monkeypatch.setenv("S12_GSTREAM_MAXB", "32")
    M, K = 300, 512
    w = _tiny_exponent_weights(M, K, 5 + B, escapes)
    p = O.pack(w)
    assert p.base_exp == -1 and (p.num_patches > 0) == escapes
    x = (O.synth_acts(B, K, 4) + np.uint16(100 << 7)).astype(np.uint16)      # activations * 2^100: products are normal fp32
    xd = dev(x)
    out = _run(eng, _cw(p), xd, M, K, B)
    assert_close(out, O.gemm_exact(w, x), what="with the CSR list")
    got = _run(eng, _cw(p), xd, M, K, B, exact=False).cpu().numpy()
    ref = O.gemm_twopass(p, x, patches=False)
    fin = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), fin)
    if escapes:
        assert not fin.all()
    assert np.abs(got[fin] - ref[fin]).max() <= REL_TOL * np.abs(ref[fin]).max()
    assert eng.device_status() == 0


@pytest.mark.parametrize("B", [8, 32])
def test_without_the_escape_list_escapes_stay_wrong(eng, O, monkeypatch, B):
    """First pass of the reference's two passes: a tensor given without its CSR list."""
    monkeypatch.setenv("S12_GSTREAM", "2")
    monkeypatch.setenv("S12_GSTREAM_MAXB", "32")
    M, K = 640, 1024
    w = O.synth_weights(M, K, 77, outlier_frac=5e-3)
    p = O.pack(w)
    x = O.synth_acts(B, K, 2)
    out = _run(eng, _cw(p), dev(x), M, K, B, exact=False)
    assert_close(out, O.gemm_twopass(p, x, patches=False), what="first pass")
    assert eng.device_status() == 0


def test_default_dispatch_takes_large_tensors(eng, O):
    """No knobs: 9000 x 4096 at B = 8 (71 row tiles) goes through the streaming kernel, and is exact."""
    M, K, B = 9000, 4096, 8
    w = O.synth_weights(M, K, 11, outlier_frac=1e-3)
    p = O.pack(w)
    x = O.synth_acts(B, K, 3)
    out = _run(eng, _cw(p), dev(x), M, K, B)
    assert eng.device_status() == 0
    assert_close(out, O.gemm_exact(w, x), what="default dispatch")


@pytest.mark.parametrize("rows,K,B", [(1024, 8192, 8), (512, 28672, 16), (4096, 14336, 32)])
def test_benchmark_shapes(eng, O, monkeypatch, rows, K, B):
    """Shapes of the 7B/8B/70B projections at the library's own choice of grid and ring."""
    monkeypatch.setenv("S12_GSTREAM", "2")
    monkeypatch.setenv("S12_GSTREAM_MAXB", "32")
    w = O.synth_weights(rows, K, rows + K + B, outlier_frac=5e-4)
    p = O.pack(w)
    x = O.synth_acts(B, K, 21)
    out = _run(eng, _cw(p, escape_table=False), dev(x), rows, K, B)
    assert eng.device_status() == 0
    assert_close(out, O.gemm_exact(w, x), what="benchmark shape")
