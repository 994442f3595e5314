import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def ofa():
    """The package (its directory name has a hyphen, hence importlib)."""
    return importlib.import_module("open-flapping-airplanes_b200")


@pytest.fixture(scope="session")
def oracle():
    from oracle import gpt_oracle
    return gpt_oracle


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
