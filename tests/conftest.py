import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def load_golden(name):
    """Return the arrays of tests/golden/<name>.npz as a dict."""
    with np.load(os.path.join(GOLDEN, name + ".npz"), allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def golden_quant():
    return load_golden("activation_quant")


@pytest.fixture(scope="session")
def golden_fused():
    return load_golden("fused_linear")


@pytest.fixture(scope="session")
def golden_pack():
    return load_golden("pack_v9_weights")


@pytest.fixture(scope="session")
def golden_nibble():
    return load_golden("nibble_pack")
