import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def rf_lib():
    """The C-ABI library, built in-tree if missing or stale (nvcc cross-compiles without a GPU)."""
    from radeonflow_kernels_b200 import _lib, build
    build.build()
    return _lib.lib()
