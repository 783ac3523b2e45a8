import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "blocks.npz")))


@pytest.fixture(scope="session")
def dev():
    """The device under test.  GPU tests fail (not skip) when the library or a device is missing:
    a silent skip would hide that the CUDA path did not run."""
    import ubridge_b200 as ub

    assert ub.lib().ub_device_count() > 0, "no CUDA device visible"
    d = ub.GcuDevice(0)
    yield d
    d.synchronize()
    assert d.device_status() == 0
