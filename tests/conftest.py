import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "sonic-moe_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_library():
    """The C-ABI shared library, (re)built in-tree if sources changed and nvcc is present."""
    sys.path.insert(0, PKG)
    import build as smoe_build

    try:
        return smoe_build.build()
    except RuntimeError:
        if os.path.exists(smoe_build.OUT):
            return smoe_build.OUT
        raise


def golden(name):
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", name + ".npz"))
