import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "server-benchmark_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "awq_golden.npz"))


@pytest.fixture(scope="session")
def built_library():
    """Path of libawq_b200.so, building it if the tree has no fresh copy."""
    import build as awq_build  # server-benchmark_b200/build.py
    return awq_build.build()
