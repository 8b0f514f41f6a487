import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) and the built CUDA library")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_fixtures.npz"))


@pytest.fixture(scope="session")
def built_lib():
    """Build the CUDA library in-tree if needed (nvcc cross-compiles without a GPU) and return its path."""
    from kiln_b200 import build
    return build.build()
