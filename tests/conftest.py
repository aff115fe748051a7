import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _ensure_library():
    """Build libso3lr_b200.so when it is missing or older than its sources (nvcc cross-compiles without a GPU)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_so3lr_b200_build", os.path.join(ROOT, "so3lr_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    try:
        mod.build()
    except Exception as e:  # a box without nvcc runs the prebuilt library
        if not os.path.exists(mod.LIB):
            raise RuntimeError(f"libso3lr_b200.so is missing and could not be built: {e}")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")
    _ensure_library()


@pytest.fixture(scope="session")
def oracle_params():
    from oracle import so3lr_oracle
    return so3lr_oracle.load_params()


@pytest.fixture(scope="session")
def reference_goldens():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_goldens.npz"))
