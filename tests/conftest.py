import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import Oracle
    return Oracle(nthreads=1)


@pytest.fixture(scope="session")
def oracle_mt():
    from oracle import Oracle
    return Oracle(nthreads=4)


@pytest.fixture(scope="session")
def gpu():
    """The product library on cuda:0. Fails (not skips) when the extension is missing on a GPU box."""
    from vpux_plugin_b200.lib import Library
    return Library(device=0)
