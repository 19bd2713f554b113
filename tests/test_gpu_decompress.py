"""Standalone decompress kernel vs the oracle: bit-exact."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, golden_packed
from gpu_util import dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from turbo_lossless_b200 import Split12Engine
    return Split12Engine()


def _cw(p, **kw):
    from turbo_lossless_b200 import CompressedWeight
    return CompressedWeight.from_packed(p, **kw)


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_cases_bit_exact(eng, O, golden, name):
    w, p = golden_packed(O, golden, name)
    cw = _cw(p)
    assert np.array_equal(_bits(eng.decompress(cw)), w)
    assert np.array_equal(_bits(eng.decompress(cw, exact=False)), O.unpack_wrong(p))


def test_every_byte_and_group(eng, O):
    """All 256 sm bytes x 16 groups, in every position of the 16-element chunk, several base_exp."""
    sm = np.repeat(np.arange(256, dtype=np.uint8), 16)
    g = np.tile(np.arange(16, dtype=np.uint8), 256)
    for shift in range(0, 16, 3):
        s2, g2 = np.roll(sm, shift), np.roll(g, shift)
        gr = (g2[0::2] | (g2[1::2] << 4)).astype(np.uint8)
        for be in (-1, 0, 1, 108, 127, 240):
            p = O.Packed(4, s2.size // 4, be, s2, gr, np.zeros(5, np.int32), np.zeros(0, np.int32),
                         np.zeros(0, np.int16), np.zeros(0, np.int16))
            assert np.array_equal(_bits(eng.decompress(_cw(p))), O.unpack_wrong(p)), (shift, be)


@pytest.mark.parametrize("M,K,frac", [(1, 2, 0.0), (3, 6, 0.3), (7, 34, 0.05), (130, 256, 1e-2),
                                      (5, 4096, 1e-3), (64, 14336, 2.5e-3)])
def test_shapes_and_tails(eng, O, M, K, frac):
    w = O.synth_weights(M, K, 100 + M + K, outlier_frac=frac)
    p = O.pack(w)
    assert np.array_equal(_bits(eng.decompress(_cw(p))), w)


def test_empty_tensor_is_a_noop(eng, O):
    from turbo_lossless_b200 import CompressedWeight
    z = torch.zeros(0, dtype=torch.uint8, device="cuda")
    cw = CompressedWeight(M=0, K=64, base_exp=100, split_sm=z, split_gr=z)
    out = torch.full((4,), 7, dtype=torch.int16, device="cuda")
    eng.decompress(cw, out=out)
    torch.cuda.synchronize()
    assert out.tolist() == [7, 7, 7, 7]


def test_config1_tensor_roundtrip(eng, O):
    """4096x4096, N(0,0.02) with 0.05% outliers x100: decompress(pack(W)) == W."""
    w = O.synth_weights(4096, 4096, 0, outlier_frac=5e-4)
    p = O.pack(w)
    got = eng.decompress(_cw(p))
    assert torch.equal(got.view(-1), dev(w).view(-1))


def test_full_size_roundtrip_on_device(eng, O):
    """lm_head-sized tensor (128256 x 4096, 0.5 G weights): the oracle packs one 4008-row slab,
    the slab is tiled on the device with per-tile CSR offsets, and the decompressed result must
    equal the tiled original bit for bit (round-trip property at full size)."""
    rows, K, tiles = 4008, 4096, 32
    w = O.synth_weights(rows, K, 5, outlier_frac=2e-4)
    p = O.pack(w)
    ro = np.concatenate([[0]] + [p.row_off[1:].astype(np.int64) + t * p.num_patches for t in range(tiles)])
    big = O.Packed(rows * tiles, K, p.base_exp, np.tile(p.sm, tiles), np.tile(p.gr, tiles),
                   ro.astype(np.int32), np.tile(p.cols, tiles), np.tile(p.correct, tiles),
                   np.tile(p.wrong, tiles))
    got = eng.decompress(_cw(big, escape_table=False))
    ref = dev(w)
    for t in range(tiles):
        assert torch.equal(got[t * rows:(t + 1) * rows], ref), t


def test_rejects_bad_arguments(eng, O):
    from turbo_lossless_b200 import CompressedWeight, S12Error
    z = torch.zeros(64, dtype=torch.uint8, device="cuda")
    with pytest.raises(S12Error):
        eng.decompress(CompressedWeight(M=3, K=7, base_exp=100, split_sm=z, split_gr=z))
