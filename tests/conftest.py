import os
import sys

import numpy as np
import pytest

# The library honours its S12_* tuning knobs only when this is set before its first launch; the tests use the
# knobs to force every kernel variant and schedule.
os.environ.setdefault("S12_TUNE", "1")

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_cuda = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_cuda = False
    if has_cuda:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def O():
    """The CPU oracle (test infrastructure)."""
    from oracle import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "split12_pack_golden.npz")
    return np.load(path)


GOLDEN_CASES = ["tiny_2x64", "odd_rows_5x130", "outliers_64x256", "wide_exponents_16x128",
                "no_escapes_8x96", "edge_columns_12x64", "base_exp_minus1_6x64"]


def golden_packed(O, golden, name):
    w = golden[name + ".w"]
    return w, O.Packed(w.shape[0], w.shape[1], int(golden[name + ".base_exp"]), golden[name + ".sm"],
                       golden[name + ".gr"], golden[name + ".row_off"], golden[name + ".cols"],
                       golden[name + ".correct"], golden[name + ".wrong"])
