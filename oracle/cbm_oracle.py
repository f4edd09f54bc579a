"""TEST INFRASTRUCTURE — CPU restatement of the reference's CBM path (builder + products).

Only ``tests/``, the smoke check and ``bench.py``'s CPU-baseline legs import this module; the
product package never does.  The compute loops live in ``cbm_oracle.c`` (loaded with ctypes); this
file restates the builder in numpy/scipy/pure Python for small inputs and wraps the C functions.

Parity status: pinned.  The reference ships no golden vectors of its own, so the pins are outputs
of the reference itself: its unmodified native source compiled into ``oracle/_ref`` (stand-in
headers for oneMKL and arbok, the sparse product forwarded to the oneMKL inside libtorch; see
``build_ref.py``) and its unmodified Python class on top.  ``tests/golden/cbm_reference.npz`` holds
such outputs for every product method; the tree updates of this file reproduce them bit for bit,
the products within the reference's own atol = rtol = 1e-4 (tests/test_matmul_correctness.py:43),
and where ``oracle/_ref`` is present the comparison is repeated live at benchmark sizes.
The tree SHAPE depends on the arborescence solver's tie-breaking (arbok upstream, unpinned there):
"parity unpinned" for the shape only; validity (``check_format``), the optimal total weight (equal
to the reference builder's) and the delta values of shared (row, parent) pairs are pinned.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from collections import deque

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, "libcbm_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_DIR, "cbm_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(src) > os.path.getmtime(_SO):
        env = {k: v for k, v in os.environ.items() if k not in ("CC", "CFLAGS")}
        subprocess.run(["make", "-C", _DIR, "-B", "libcbm_oracle.so"], check=True, env=env,
                       capture_output=True)
    return _SO


def clib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_max_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


# ----------------------------------------------------------------------------------------------
# Builder restatement (small inputs)
# ----------------------------------------------------------------------------------------------
def pattern_rows(edge_index: np.ndarray, n: int) -> list[np.ndarray]:
    """Sorted column list of every row (the CSR the reference gets from MKL, cbm_extensions.cpp:15-43)."""
    rows = [[] for _ in range(n)]
    for r, c in zip(edge_index[0].tolist(), edge_index[1].tolist()):
        rows[r].append(c)
    return [np.unique(np.asarray(r, dtype=np.int64)) for r in rows]


def candidate_edges(edge_index: np.ndarray, n: int, alpha: int) -> list[tuple[int, int, int]]:
    """Distance graph G as (src, dst, weight), in the reference's order
    (cbm/cbm_extensions.cpp:75-102): for every row the virtual edge (n -> row, |row|), then for every
    later row sharing a column (the upper triangle of A*A^T, diagonal skipped) up to two edges."""
    import scipy.sparse as sp
    a = sp.csr_matrix((np.ones(edge_index.shape[1], dtype=np.int64), (edge_index[0], edge_index[1])),
                      shape=(n, n))
    a.data[:] = 1
    inter = sp.triu(a @ a.T, k=1).tocsr()
    nnz = np.diff(a.indptr)
    g = []
    for row in range(n):
        g.append((n, row, int(nnz[row])))
        for k in range(inter.indptr[row], inter.indptr[row + 1]):
            col, val = int(inter.indices[k]), int(inter.data[k])
            h = int(nnz[row] + nnz[col] - 2 * val)
            if h < nnz[row] - alpha:
                g.append((col, row, h))
            if h < nnz[col] - alpha:
                g.append((row, col, h))
    return g


def min_arborescence(n_vertices: int, root: int, edges: list[tuple[int, int, int]]) -> dict[int, tuple[int, int]]:
    """Chu-Liu/Edmonds minimum-cost arborescence, recursive contraction form, O(V*E): the published
    algorithm the reference obtains from arbok::TarjanPQ (cbm/cbm_extensions.cpp:109-148).
    Returns {vertex: (parent, weight)} for every vertex but the root."""
    best: dict[int, tuple[int, int, int]] = {}
    for idx, (u, v, w) in enumerate(edges):
        if u == v or v == root:
            continue
        if v not in best or w < edges[best[v][2]][2]:
            best[v] = (u, w, idx)
    # find a cycle among the chosen edges
    color: dict[int, int] = {}
    cycle = None
    for s in best:
        if s in color:
            continue
        path = []
        x = s
        while x in best and x not in color:
            color[x] = s
            path.append(x)
            x = best[x][0]
        if x in best and color.get(x) == s:
            cycle = path[path.index(x):]
            break
    if cycle is None:
        return {v: (u, w) for v, (u, w, _) in best.items()}
    cyc = set(cycle)
    super_v = n_vertices
    new_edges, origin = [], []
    for idx, (u, v, w) in enumerate(edges):
        if u in cyc and v in cyc:
            continue
        if v in cyc:
            new_edges.append((u, super_v, w - best[v][1]))
        elif u in cyc:
            new_edges.append((super_v, v, w))
        else:
            new_edges.append((u, v, w))
        origin.append(idx)
    sub = min_arborescence(n_vertices + 1, root, new_edges)
    # map the contracted solution back to original edges
    result: dict[int, tuple[int, int]] = {}
    chosen_by_pair: dict[tuple[int, int, int], int] = {}
    for j, e in enumerate(new_edges):
        chosen_by_pair.setdefault(e, origin[j])
    for v, (u, w) in sub.items():
        ou, ov, ow = edges[chosen_by_pair[(u, v, w)]]
        result[ov] = (ou, ow)
    entered = next(ov for ov in result if ov in cyc)
    for v in cycle:
        if v != entered:
            result[v] = (best[v][0], best[v][1])
    return result


def build_structure(edge_index: np.ndarray, alpha: int, col_mul: np.ndarray | None = None,
                    parent: np.ndarray | None = None) -> dict:
    """Tree + deltas following cbm/cbm_extensions.cpp:150-286 (v1) / :468-604 (v2): breadth-first
    traversal from the virtual root, sorted-merge deltas (+1 only-in-child, -1 only-in-parent,
    scaled by ``col_mul[col]`` for v2), tree CSR.  ``parent`` may be supplied to reuse a tree."""
    n = int(edge_index.max()) + 1 if edge_index.size else 0
    rows = pattern_rows(edge_index, n)
    if parent is None:
        sol = min_arborescence(n + 1, n, candidate_edges(edge_index, n, alpha))
        parent = np.array([sol[v][0] for v in range(n)], dtype=np.int64)
    children = [[] for _ in range(n + 1)]
    for v in range(n):
        children[int(parent[v])].append(v)
    d_row, d_col, d_val = [], [], []
    order = []
    queue = deque([n])
    while queue:
        u = queue.popleft()
        for v in children[u]:
            queue.append(v)
            order.append(v)
            cv = rows[v]
            if u == n:
                plus, minus = cv, np.empty(0, dtype=np.int64)
            else:
                cu = rows[u]
                plus, minus = np.setdiff1d(cv, cu, assume_unique=True), np.setdiff1d(cu, cv, assume_unique=True)
            for c in plus.tolist():
                d_row.append(v); d_col.append(c); d_val.append(1.0 if col_mul is None else float(col_mul[c]))
            for c in minus.tolist():
                d_row.append(v); d_col.append(c); d_val.append(-1.0 if col_mul is None else -float(col_mul[c]))
    mst_row = np.zeros(n + 2, dtype=np.int32)
    for u in range(n + 1):
        mst_row[u + 1] = mst_row[u] + len(children[u])
    mst_col = np.array([v for u in range(n + 1) for v in children[u]], dtype=np.int32)
    # COO -> CSR sorted by (row, col) as torch's coalesce does (cbm/cbm.py:120-141)
    d_row, d_col, d_val = np.asarray(d_row, np.int64), np.asarray(d_col, np.int64), np.asarray(d_val, np.float32)
    o = np.lexsort((d_col, d_row))
    d_row, d_col, d_val = d_row[o], d_col[o], d_val[o]
    crow = np.zeros(n + 1, dtype=np.int32)
    np.add.at(crow, d_row + 1, 1)
    crow = np.cumsum(crow).astype(np.int32)
    return dict(n=n, parent=parent.astype(np.int32), mst_row=mst_row, mst_col=mst_col, crow=crow,
                col=d_col.astype(np.int32), val=d_val, weight=int(d_col.shape[0]), bfs=order)


def reconstruct_rows(n, mst_row, mst_col, crow, col, val) -> list[set]:
    """The validator of cbm/cbm.py:69-115: every row's column set from the tree and the deltas."""
    s = [set() for _ in range(n + 1)]
    queue = deque([n])
    seen = set()
    while queue:
        u = queue.popleft()
        if u in seen:
            continue
        seen.add(u)
        for v in mst_col[mst_row[u]:mst_row[u + 1]].tolist():
            queue.append(v)
            s[v].update(s[u])
            for c, w in zip(col[crow[v]:crow[v + 1]].tolist(), val[crow[v]:crow[v + 1]].tolist()):
                if w > 0:
                    s[v].add(c)
                elif w < 0:
                    s[v].remove(c)
                else:
                    raise ValueError("zero delta value")
    if len(seen) != n + 1:
        raise ValueError("tree does not reach every row")
    return s[:n]


# ----------------------------------------------------------------------------------------------
# Products (C restatement)
# ----------------------------------------------------------------------------------------------
def _c32(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def csr_spmm(crow, col, val, x, parallel=False) -> np.ndarray:
    """seq_/omp_s_spmm_csr_int32 (cbm/cbm_extensions.cpp:790-843, 1707-1755)."""
    crow, col, val, x = _c32(crow, np.int32), _c32(col, np.int32), _c32(val, np.float32), _c32(x, np.float32)
    n, f = crow.shape[0] - 1, x.shape[1]
    y = np.empty((n, f), dtype=np.float32)
    row_b, row_e = np.ascontiguousarray(crow[:-1]), np.ascontiguousarray(crow[1:])
    clib().oracle_csr_spmm(n, _p(row_b), _p(row_e), _p(col), _p(val), _p(x), f, _p(y), int(parallel))
    return y


def update(mst_row, mst_col, y, parallel=False) -> np.ndarray:
    """In place: seq_/omp_s_update_csr_int32 (cbm/cbm_extensions.cpp:742-786, 1485-1610)."""
    mst_row, mst_col = _c32(mst_row, np.int32), _c32(mst_col, np.int32)
    assert y.dtype == np.float32 and y.flags.c_contiguous
    n, f = y.shape
    if clib().oracle_update(n, _p(mst_row), _p(mst_col), _p(y), f, int(parallel)):
        raise MemoryError("oracle_update")
    return y


def fused_update(mst_row, mst_col, mult, y, parallel=False) -> np.ndarray:
    """In place: seq_/omp_s_fused_update_csr_int32 (cbm/cbm_extensions.cpp:998-1105, 1376-1483)."""
    mst_row, mst_col, mult = _c32(mst_row, np.int32), _c32(mst_col, np.int32), _c32(mult, np.float32)
    assert y.dtype == np.float32 and y.flags.c_contiguous
    n, f = y.shape
    if clib().oracle_fused_update(n, _p(mst_row), _p(mst_col), _p(mult), _p(y), f, int(parallel)):
        raise MemoryError("oracle_fused_update")
    return y


def spmm_update(mst_row, mst_col, crow, col, val, x, parallel=False) -> np.ndarray:
    """seq_/omp_s_spmm_update_csr_int32 (cbm/cbm_extensions.cpp:650-740, 1108-1219)."""
    return update(mst_row, mst_col, csr_spmm(crow, col, val, x, parallel), parallel)


def fused_spmm_update(mst_row, mst_col, crow, col, val, mult, x, parallel=False) -> np.ndarray:
    """seq_/omp_s_fused_spmm_update_csr_int32 (cbm/cbm_extensions.cpp:845-996, 1224-1374)."""
    return fused_update(mst_row, mst_col, mult, csr_spmm(crow, col, val, x, parallel), parallel)


def dense_adjacency(edge_index: np.ndarray, n: int) -> np.ndarray:
    a = np.zeros((n, n), dtype=np.float64)
    a[edge_index[0], edge_index[1]] = 1.0
    return a


def row_multiplier(edge_index: np.ndarray, n: int) -> np.ndarray:
    """D^-1/2 from row degrees as cbm/cbm.py:34-41 computes it (fp32, inf for an empty row)."""
    deg = np.bincount(edge_index[0], minlength=n).astype(np.float32)
    with np.errstate(divide="ignore"):
        return np.power(deg, np.float32(-0.5), dtype=np.float32)
