import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def ref_pins():
    return np.load(os.path.join(GOLDEN, "ref_pins.npz"))


@pytest.fixture(scope="session")
def oracle_cases():
    return np.load(os.path.join(GOLDEN, "oracle_cases.npz"))


@pytest.fixture(scope="session")
def dgq():
    """The C-ABI library through its ctypes binding; GPU tests only."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from distributed_gptq_b200 import _C
    return _C
