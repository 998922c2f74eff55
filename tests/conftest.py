"""pytest configuration: registers the ``gpu`` marker and puts the repository root on sys.path.

``-m "not gpu"`` tests run on a machine without a GPU (oracle vs. golden vectors, host logic,
C-ABI symbol checks, two-rank gloo tests); ``-m gpu`` tests are the parity tests proper."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
