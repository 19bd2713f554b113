"""Device packer vs the oracle packer (itself pinned to the reference's CPU packer): identical bytes."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, golden_packed
from gpu_util import dev

pytestmark = pytest.mark.gpu
FIELDS = (("split_sm", "sm"), ("split_gr", "gr"), ("row_offsets", "row_off"), ("patch_cols", "cols"),
          ("patch_correct", "correct"), ("patch_wrong", "wrong"))


def _check(cw, ref):
    assert (cw.M, cw.K, cw.base_exp, cw.num_patches) == (ref.M, ref.K, ref.base_exp, ref.num_patches)
    for a, b in FIELDS:
        t = getattr(cw, a)
        if t is None:
            assert ref.num_patches == 0
            continue
        assert np.array_equal(t.cpu().numpy(), getattr(ref, b)), a


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_cases(O, golden, name):
    from turbo_lossless_b200 import CompressedWeight
    w, ref = golden_packed(O, golden, name)
    _check(CompressedWeight.pack_on_device(dev(w)), ref)


@pytest.mark.parametrize("M,K,frac", [(4096, 4096, 5e-4), (3000, 1056, 2e-2), (1, 32, 0.0), (5000, 14336, 2.5e-3)])
def test_matches_oracle_packer(O, M, K, frac):
    from turbo_lossless_b200 import CompressedWeight
    w = O.synth_weights(M, K, M + K, outlier_frac=frac)
    _check(CompressedWeight.pack_on_device(dev(w)), O.pack(w))


def test_pack_then_decompress_roundtrip_full_size():
    """lm_head-sized (128256 x 4096) random bf16 weights generated on the device: pack, decompress,
    compare bit for bit -- the round-trip property at full size, without any host copy."""
    from turbo_lossless_b200 import CompressedWeight, Split12Engine
    g = torch.Generator(device="cuda").manual_seed(1)
    w = (torch.randn(128256, 4096, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    cw = CompressedWeight.pack_on_device(w)
    assert 0 < cw.num_patches < 0.001 * w.numel()
    out = Split12Engine().decompress(cw)
    assert torch.equal(out, w.view(torch.int16))


def test_pack_under_dependent_launch(O, golden):
    """The packer's five kernels each consume their predecessor's output; with programmatic dependent launch
    enabled every one of them waits for it before reading."""
    from turbo_lossless_b200 import CompressedWeight, Split12Engine
    eng = Split12Engine()
    old = eng.set_dependent_launch(True)
    try:
        for name in GOLDEN_CASES:
            w, ref = golden_packed(O, golden, name)
            _check(CompressedWeight.pack_on_device(dev(w)), ref)
        w = O.synth_weights(3000, 4096, 3, outlier_frac=1e-2)
        for _ in range(3):
            _check(CompressedWeight.pack_on_device(dev(w)), O.pack(w))
    finally:
        eng.set_dependent_launch(old)
