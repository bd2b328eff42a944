import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def tt():
    """The product package (its directory name has a hyphen, hence importlib)."""
    return importlib.import_module("pku-aiprogramming_b200")


@pytest.fixture(scope="session")
def oracle():
    from oracle import attention_oracle
    return attention_oracle
