import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "deepseek-v3_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_cpu():
    import numpy as np
    return np.load(os.path.join(GOLDEN, "ref_cpu_interp.npz"))


@pytest.fixture(scope="session")
def golden_gpu():
    import numpy as np
    path = os.path.join(GOLDEN, "ref_gpu_triton.npz")
    if not os.path.exists(path):
        pytest.skip("GPU-generated golden vectors not present")
    return np.load(path)
