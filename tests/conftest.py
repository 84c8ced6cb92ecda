import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line(
        "markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as oracle_module
    oracle_module.build()
    return oracle_module


@pytest.fixture(scope="session")
def mgpu():
    """The ctypes binding with the library loaded; fails loudly if it is not
    built (no CPU fallback exists)."""
    import moderngpu_b200
    moderngpu_b200.load_library()
    return moderngpu_b200
