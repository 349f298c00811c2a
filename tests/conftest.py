import os
import sys

import pytest

# validation mode: device status words are read back after every call and outputs start as NaN
os.environ.setdefault("EASYMLX_B200_CHECK", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def golden_path(name):
    return os.path.join(ROOT, "tests", "golden", name + ".npz")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    def load(name):
        with np.load(golden_path(name)) as f:
            return {k: f[k] for k in f.files}

    return load
