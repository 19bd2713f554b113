"""The CPU oracle against the golden vectors produced by the unmodified reference packer."""
import hashlib

import numpy as np
import pytest

from conftest import GOLDEN_CASES, golden_packed

FIELDS = ("sm", "gr", "row_off", "cols", "correct", "wrong")


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_pack_matches_reference_golden(O, golden, name):
    w, ref = golden_packed(O, golden, name)
    assert O.find_base_exp(w) == ref.base_exp
    mine = O.pack(w)
    for f in FIELDS:
        assert np.array_equal(getattr(mine, f), getattr(ref, f)), f


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_unpack_roundtrip_is_lossless(O, golden, name):
    w, ref = golden_packed(O, golden, name)
    assert np.array_equal(O.unpack_exact(ref), w)
    assert np.array_equal(O.unpack_numpy(ref, exact=True), w)
    assert np.array_equal(O.unpack_numpy(ref, exact=False), O.unpack_wrong(ref))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_patch_wrong_is_the_group0_decode(O, golden, name):
    """patch_wrong = sign<<15 | base_exp<<7 | mantissa (split12_pack.c:117-122) must be what the
    element decode yields for group 0."""
    w, ref = golden_packed(O, golden, name)
    if ref.num_patches == 0:
        return
    wrong = O.unpack_wrong(ref)
    rows = np.repeat(np.arange(ref.M), np.diff(ref.row_off))
    assert np.array_equal(wrong[rows, ref.cols], ref.wrong.view(np.uint16))
    assert np.array_equal(w[rows, ref.cols], ref.correct.view(np.uint16))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_csr_invariants(O, golden, name):
    _, ref = golden_packed(O, golden, name)
    assert ref.row_off[0] == 0 and ref.row_off[-1] == ref.num_patches
    assert np.all(np.diff(ref.row_off) >= 0)
    for r in range(ref.M):
        c = ref.cols[ref.row_off[r]:ref.row_off[r + 1]]
        assert np.all(np.diff(c) > 0)


def test_config1_digests(O, golden):
    """The 4096x4096 benchmark tensor: same digests as the reference packer produced."""
    w = O.synth_weights(4096, 4096, 0, outlier_frac=5e-4)
    p = O.pack(w)
    dig = [hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
           for a in (w, p.sm, p.gr, p.row_off, p.cols, p.correct, p.wrong)]
    assert dig == list(golden["config1.digests"])
    assert [p.base_exp, p.num_patches] == list(golden["config1.meta"])
    assert np.array_equal(O.unpack_exact(p), w)


def test_compiled_reference_packer_when_present(O, golden):
    if not O.have_ref_packer():
        pytest.skip("oracle/_ref not built (no upstream checkout at build time)")
    for name in GOLDEN_CASES:
        w, ref = golden_packed(O, golden, name)
        got = O.pack(w, use_ref=True)
        assert got.base_exp == ref.base_exp
        for f in FIELDS:
            assert np.array_equal(getattr(got, f), getattr(ref, f)), (name, f)


def test_all_sm_bytes_and_groups(O):
    """Every (sm byte, group) pair decodes as the formula says, for several base_exp."""
    sm = np.repeat(np.arange(256, dtype=np.uint8), 16)
    g = np.tile(np.arange(16, dtype=np.uint8), 256)
    gr = (g[0::2] | (g[1::2] << 4)).astype(np.uint8)
    for be in (-1, 0, 108, 240):
        p = O.Packed(1, sm.size, be, sm, gr, np.zeros(2, np.int32), np.zeros(0, np.int32),
                     np.zeros(0, np.int16), np.zeros(0, np.int16))
        got = O.unpack_wrong(p).ravel()
        exp = ((((sm.astype(np.int64) >> 7) << 15) | ((be + g.astype(np.int64)) << 7) | (sm & 0x7F)) & 0xFFFF)
        assert np.array_equal(got, exp.astype(np.uint16))
