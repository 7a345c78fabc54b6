import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the kernels through the C ABI)")


@pytest.fixture(scope="session")
def drkv_lib():
    """libdrkv.so, built in-tree if missing or stale."""
    from deusridet_b200 import build, capi
    build.build()
    return capi.load_library()


@pytest.fixture(scope="session")
def oracle():
    from oracle import cbind
    cbind.lib()
    return cbind
