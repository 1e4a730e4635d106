import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# every communicator of the test suite carries the debug guard behind its staging layout: a
# kernel (or host executor) that writes out of bounds fails the test at pause or destroy
os.environ.setdefault("AMEM_CANARY", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    # tests/test_zz_* files are meant to run after everything else
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz"), ))


@pytest.fixture(scope="session")
def lib():
    from asystem_amem_b200 import load_library
    return load_library()
