import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    """CPU oracle (test infrastructure)."""
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def gk():
    """The product package (directory name carries a hyphen, so import it by string)."""
    return importlib.import_module("gllm-kernels_b200")
