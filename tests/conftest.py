import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(autouse=True)
def _seeded_torch():
    """Every test draws the same torch random numbers on every run (host and device generators)."""
    import torch
    torch.manual_seed(20240)
    yield


@pytest.fixture(scope="session")
def port():
    from oracle.oracle import CpuOracle
    return CpuOracle("port")


@pytest.fixture(scope="session")
def ref():
    from oracle.oracle import CpuOracle, available
    if not available("ref"):
        pytest.skip("compiled reference (oracle/_ref) not present")
    return CpuOracle("ref")


@pytest.fixture(scope="session")
def lib():
    from libmolgrid_b200 import build
    build.build_library()
    from libmolgrid_b200 import _cabi
    return _cabi.lib()
