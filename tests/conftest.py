import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "project-aeon_b200"))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def pytest_collection_modifyitems(config, items):
    # A GPU-marked test on a machine without a device is an error of selection, not a skip:
    # the driver selects with -m "not gpu" here and -m gpu on the box.
    pass


@pytest.fixture(scope="session")
def oracle():
    import oracle_py
    return oracle_py
