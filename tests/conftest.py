import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def device():
    """One library context on GPU 0 for the whole session (like Device::test_instance in the reference)."""
    import floneum_b200
    return floneum_b200.Device.gpu(0)


# tolerance of the path: outputs vs the f32 oracle on the same (bf16-rounded) inputs
MAX_ABS_TOL = 2e-3
MEAN_ABS_TOL = 2e-4


def assert_close(got, want, max_tol=MAX_ABS_TOL, mean_tol=MEAN_ABS_TOL, what=""):
    import numpy as np
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - want)
    assert err.max() <= max_tol, f"{what}: max-abs error {err.max():.3e} > {max_tol}"
    assert err.mean() <= mean_tol, f"{what}: mean-abs error {err.mean():.3e} > {mean_tol}"
