import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "cbm_small.npz"))


def golden_case(golden, k):
    return (golden[f"case{k}_edge_index"].astype(np.int64), golden[f"case{k}_x"], golden[f"case{k}_y"],
            golden[f"case{k}_y_norm"])
