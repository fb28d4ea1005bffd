import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def rel_err_ok(x, ref, tol):
    """|x - ref| <= tol * (|ref| + rms(ref)) elementwise; returns (ok, worst ratio)."""
    import numpy as np
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    bound = tol * (np.abs(ref) + rms) + 1e-30
    ratio = np.abs(x - ref) / bound
    worst = float(ratio.max()) if ratio.size else 0.0
    return bool(worst <= 1.0) and bool(np.isfinite(x).all()), worst


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    o.lib()
    return o
