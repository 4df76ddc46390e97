import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def normwise(a, b):
    """max|a - b| / max|b| -- the tolerance form used for every floating-point comparison."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    if b.size == 0:
        return 0.0
    scale = np.abs(b).max()
    return float(np.abs(a - b).max() / scale) if scale > 0 else float(np.abs(a - b).max())


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return dict(np.load(os.path.join(GOLDEN, name)))
    return load


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    if not oracle.available("port"):
        oracle.build()
    return oracle


@pytest.fixture(autouse=True)
def _no_stale_device_status(request):
    """After every GPU test the device status word must be clear: a kernel that reported a bad
    index, a bad element or a timeout is pinned on the test that ran it, not on a later one.
    Tests that provoke a report on purpose read (and thereby clear) it themselves."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from khan_b200 import ani_mod
    status = ani_mod.device_status()
    assert status == 0, f"{request.node.name} left device status {status}"
