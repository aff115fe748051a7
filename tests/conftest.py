import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle_params():
    from oracle import so3lr_oracle
    return so3lr_oracle.load_params()


@pytest.fixture(scope="session")
def reference_goldens():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_goldens.npz"))
