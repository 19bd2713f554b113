"""Helpers shared by the GPU parity tests (all device work goes through the C ABI)."""
import numpy as np
import torch

# fp32-accumulate outputs: max |y - ref| / max |ref|.  The specification asks for <= 1e-2;
# the kernels are held to 1e-4 (observed ~1e-6) so that a wrong escape or a dropped column shows.
REL_TOL = 1e-4


def dev(a: np.ndarray) -> torch.Tensor:
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    scale = float(np.max(np.abs(ref))) or 1.0
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)))) / scale


def assert_close(got, ref, tol=REL_TOL, what=""):
    if isinstance(got, torch.Tensor):
        got = got.detach().cpu().numpy()
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    e = rel_err(got, ref)
    assert e <= tol, f"{what}: rel err {e:.3e} > {tol:.1e}"
    return e
