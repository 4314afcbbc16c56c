import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_cpu_vectors.npz"))


@pytest.fixture(scope="session")
def built_lib():
    """The in-tree CUDA library, built on demand (nvcc cross-compiles without a GPU)."""
    from colinfer_b200 import build
    return build.build()
