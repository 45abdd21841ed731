import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.loader import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle.loader import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libref_attn.so not built (needs the reference tree at build time)")
    return Reference()


@pytest.fixture(scope="session")
def seeded():
    return np.load(os.path.join(GOLDEN, "ref_seeded.npz"))


def rel_err(a, b):
    """max|a-b| / max|b| per tensor: the fp32 parity measure."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
