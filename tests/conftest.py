import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (built on demand with make); test infrastructure only."""
    from tests import harness

    return harness.load_oracle()


@pytest.fixture(scope="session")
def libs():
    """Paths of the built CUDA libraries (built on demand with nvcc)."""
    from texo_b200 import build

    return build.build()
