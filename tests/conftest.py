import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module("knivesysl-xe_b200")


@pytest.fixture(scope="session")
def wl():
    return importlib.import_module("knivesysl-xe_b200.workloads")


@pytest.fixture(scope="session")
def lib(pkg):
    """The CUDA library bound to device 0; GPU tests fail (not skip) if it cannot load."""
    build = importlib.import_module("knivesysl-xe_b200.build")
    build.build()
    L = pkg.load()
    assert L.tq_set_device(0) == 0
    return L
