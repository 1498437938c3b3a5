import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def rel_err(a, b):
    """The reference's error metric: max|a-b| / max(max|b|, 1e-9) (rust/src/main.rs:814-820)."""
    import numpy as np

    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-9))


@pytest.fixture(scope="session")
def orc():
    import oracle

    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def gpu():
    """The library's context on cuda:0. Fails loudly when the CUDA library is absent."""
    import asca_b200

    g = asca_b200.Gpu(0)
    # the tests mix torch kernels (casts, transposes, clones) with the library's: one stream, so that they are ordered
    g.use_torch_stream()
    return g
