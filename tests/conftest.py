import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "llm-scaler_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    def load(name):
        return np.load(os.path.join(GOLDEN, name + ".npz"))
    return load


@pytest.fixture(scope="session")
def lib_built():
    """Builds libb2q.so if it is missing (nvcc cross-compiles without a GPU)."""
    so = os.path.join(PKG, "custom_esimd_kernels_vllm", "libb2q.so")
    if not os.path.exists(so):
        sys.path.insert(0, PKG)
        import build as b2q_build
        b2q_build.build()
    return so
