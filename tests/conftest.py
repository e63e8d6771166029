import os
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device; run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


@pytest.fixture(scope="session")
def dev():
    """The opened device.  GPU tests fail (not skip) when the library or the device is missing:
    a silent skip would hide a fallback."""
    import vernondsl_b200 as vd

    d = vd.Device(0)
    yield d
    d.close()


@pytest.fixture()
def stream(dev):
    s = dev.stream()
    yield s
    s.close()
