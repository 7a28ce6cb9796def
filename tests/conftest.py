import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # a GPU test on a box without a device is a hard error of the environment, not a skip: the default
    # CPU run deselects them with -m "not gpu".
    pass


@pytest.fixture(scope="session")
def lib():
    from refactorgraph_b200 import capi
    return capi.load()
