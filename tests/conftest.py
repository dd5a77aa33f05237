import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc

    orc.lib()
    return orc


@pytest.fixture(scope="session")
def backend():
    """One CUDA context for the GPU tests; creating it fails loudly without a B200."""
    import prism_engine_b200 as p

    be = p.CudaBackend(device=0)
    yield be
    be.close()


def rel_l2(got_bits, want_bits):
    import numpy as np

    g = np.asarray(got_bits, np.uint16).view(np.float16).astype(np.float64)
    w = np.asarray(want_bits, np.uint16).view(np.float16).astype(np.float64)
    d = np.linalg.norm(w)
    return float(np.linalg.norm(g - w) / (d if d > 0 else 1.0))
