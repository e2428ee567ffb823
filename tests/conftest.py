import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from checkers import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def lib():
    """The product library; built on first use if the .so is missing (CPU-only boxes included)."""
    from proteinpredictmachinelearning_b200 import LIB_PATH, load
    if not os.path.exists(LIB_PATH):
        from proteinpredictmachinelearning_b200.build import build
        build()
    return load()
