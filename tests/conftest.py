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


class ReferenceGolden:
    """``tests/golden/cbm_reference.npz``: arrays the reference itself produced (generator:
    tests/golden/make_golden_ref.py).  Bit-identical arrays are stored once; ``aliases`` maps the
    other keys to the stored copy."""

    def __init__(self, path):
        import json
        self._z = np.load(path)
        self._alias = json.loads(str(self._z["aliases"]))
        self.names = [str(s) for s in self._z["names"]]

    def __contains__(self, key):
        return key in self._alias or key in self._z.files

    def __getitem__(self, key):
        return self._z[self._alias.get(key, key)]

    def case(self, name, normalized):
        tag = "norm" if normalized else "plain"
        prefix = f"{name}/{tag}/"
        keys = [k[len(prefix):] for k in list(self._z.files) + list(self._alias) if k.startswith(prefix)]
        d = {k: self[prefix + k] for k in keys}
        d["x"] = self[f"{name}/x"]
        d["alpha"] = int(self[f"{name}/alpha"])
        return d


@pytest.fixture(scope="session")
def ref_golden():
    return ReferenceGolden(os.path.join(ROOT, "tests", "golden", "cbm_reference.npz"))
