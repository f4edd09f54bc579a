"""Generates the committed fixtures ``cbm_small.npz``.

The reference holds no golden vectors for the CBM product: its tests compare against
``torch.sparse`` on Erdős–Rényi graphs with 25 nodes, p = 0.5 / 0.75, F = 10 and integer-valued
features (tests/test_matmul_correctness.py:11-61, tests/test_message_passing.py:39-43), and the
reference cannot be imported offline (its native module needs oneMKL and arbok).  The fixtures are
therefore produced by the same check the reference applies to itself: graphs of that shape with
integer features, and ``Y = A @ X`` / ``Y = D^-1/2 (A+I) D^-1/2 @ X`` evaluated densely in float64.
The unnormalized outputs are exact integers, so they pin a float32 implementation bit for bit.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from cbm4gnn_b200 import graphs  # noqa: E402


def main():
    out = {}
    cases = [(25, 0.5, 10, 0), (25, 0.5, 10, 1), (25, 0.75, 10, 2), (40, 0.3, 7, 3), (64, 0.2, 47, 4)]
    for k, (n, p, f, seed) in enumerate(cases):
        ei = graphs.erdos_renyi(n, p, 7000 + seed)
        n_eff = int(ei.max()) + 1
        rng = np.random.default_rng(8000 + seed)
        x = rng.integers(0, 10, size=(n_eff, f)).astype(np.float32)
        a = np.zeros((n_eff, n_eff))
        a[ei[0], ei[1]] = 1.0
        y = a @ x.astype(np.float64)
        a_loop = a.copy()
        np.fill_diagonal(a_loop, 1.0)
        s = a_loop.sum(1) ** -0.5
        y_norm = (s[:, None] * a_loop * s[None, :]) @ x.astype(np.float64)
        out[f"case{k}_edge_index"] = ei.astype(np.int32)
        out[f"case{k}_x"] = x
        out[f"case{k}_y"] = y.astype(np.float32)
        out[f"case{k}_y_norm"] = y_norm
    out["n_cases"] = np.array(len(cases))
    np.savez_compressed(os.path.join(os.path.dirname(__file__), "cbm_small.npz"), **out)


if __name__ == "__main__":
    main()
