"""Shared helpers of the test-suite (CPU side)."""
import numpy as np
import torch

from cbm4gnn_b200.utility import add_self_loops


def with_self_loops(ei: np.ndarray) -> np.ndarray:
    return add_self_loops(torch.from_numpy(ei)).numpy()


def dense_product(ei: np.ndarray, x: np.ndarray, normalized: bool) -> np.ndarray:
    """float64 ``A @ x`` or ``D^-1/2 A D^-1/2 @ x`` (D = row degrees of the matrix as given)."""
    n = x.shape[0]
    a = np.zeros((n, n))
    a[ei[0], ei[1]] = 1.0
    if normalized:
        with np.errstate(divide="ignore"):
            s = a.sum(1) ** -0.5
        a = s[:, None] * a * s[None, :]
    return a @ x.astype(np.float64)


def sparse_product(ei: np.ndarray, x: np.ndarray, normalized: bool) -> np.ndarray:
    """The same through scipy CSR in float64, for sizes a dense matrix does not fit."""
    import scipy.sparse as sp
    n = x.shape[0]
    a = sp.csr_matrix((np.ones(ei.shape[1]), (ei[0], ei[1])), shape=(n, n))
    if normalized:
        s = np.asarray(a.sum(1)).ravel() ** -0.5
        a = sp.diags(s) @ a @ sp.diags(s)
    return a @ x.astype(np.float64)
