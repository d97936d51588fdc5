import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_pkg():
    """The package directory carries the reference's name with a hyphen, so it is imported through importlib."""
    return importlib.import_module("ameva-compute_b200")


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()
