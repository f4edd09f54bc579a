"""The host-side schedule of a plan (no GPU): sizes and the pre-launch checks."""
import ctypes

import numpy as np
import pytest
import torch

from cbm4gnn_b200 import _lib, graphs
from cbm4gnn_b200.cbm import cbm_matrix
from cbm4gnn_b200.sharding import partition_subtrees
from helpers import with_self_loops


def _cbm(ei, alpha=0, normalized=False):
    e = torch.from_numpy(np.ascontiguousarray(ei)).to(torch.int32)
    return cbm_matrix(e, torch.ones(e.shape[1]), alpha=alpha, normalized=normalized)


def _schedule(c, perm=None, n_labels=0, own=None, mst_col=None):
    L = _lib.lib()
    n = c.num_rows
    p = lambda a: None if a is None else ctypes.c_void_p(a.ctypes.data)
    out = [ctypes.c_int32() for _ in range(4)]
    mult = None if c.col_multiplier is None else c.col_multiplier.numpy()
    mc = c.mst_col.numpy() if mst_col is None else mst_col
    b, e = own if own else (0, n_labels or n)
    perm32 = None if perm is None else np.ascontiguousarray(perm, dtype=np.int32)
    rc = L.cbm_b200_schedule_info(n, p(c.mst_row.numpy()), p(mc), p(c._crow), p(c._dcol), p(c._dval), p(mult),
                                  p(perm32), n_labels, b, e, *[ctypes.byref(o) for o in out])
    return rc, [o.value for o in out]


def _expected(c, rows=None):
    dl = np.diff(c._crow)
    rows = np.arange(c.num_rows) if rows is None else rows
    split = dl[rows] > 192
    n_partial = int((-(-dl[rows][split] // 128) - 1).sum())
    easy = int(((c._parent[rows] == c.num_rows) & ~split).sum())
    return len(rows) + n_partial, n_partial + easy, n_partial, len(rows)


@pytest.mark.parametrize("make", [
    lambda: _cbm(graphs.erdos_renyi(25, 0.5, 1), 2),
    lambda: _cbm(graphs.make_graph("c1"), 0),
    lambda: _cbm(with_self_loops(graphs.make_graph("c1", scale=0.5)), 1, normalized=True),
    lambda: _cbm(with_self_loops(graphs.copy_model(2000, 0.95, 20, 3)), 4, normalized=True),
])
def test_schedule_sizes_and_checks(make):
    c = make()
    rc, got = _schedule(c)
    assert rc == 0, _lib.lib().cbm_b200_last_error()
    assert tuple(got) == _expected(c)


def test_schedule_of_a_chain_and_of_a_hub():
    n = 600
    rows = np.repeat(np.arange(n), np.arange(1, n + 1))
    cols = np.concatenate([np.arange(i + 1) for i in range(n)])
    c = _cbm(np.stack([rows, cols]), 0)                 # one chain of depth n: nothing but waiting items
    rc, got = _schedule(c)
    assert rc == 0 and tuple(got) == (n, 1, 0, n)
    c = _cbm(np.stack([rows, cols]), 100000)            # no compression: long rows are split
    rc, got = _schedule(c)
    assert rc == 0 and tuple(got) == _expected(c) and got[2] > 0


def test_schedule_of_shards_and_refusals():
    c = _cbm(with_self_loops(graphs.make_graph("c1")), 0, normalized=True)
    n = c.num_rows
    part = partition_subtrees(c, 3)
    total_rows = 0
    for g in range(3):
        rc, got = _schedule(c, perm=part.perm, n_labels=part.n_labels, own=part.offsets(g))
        assert rc == 0, _lib.lib().cbm_b200_last_error()
        mine = np.nonzero(part.perm // part.shard_rows == g)[0]
        assert tuple(got) == _expected(c, mine)
        total_rows += got[3]
    assert total_rows == n
    # an owned range that cuts a subtree
    deep = int(np.nonzero(c._parent != n)[0][0])
    rc, _ = _schedule(c, perm=np.arange(n), n_labels=n, own=(deep, deep + 1))
    assert rc == 1 and b"cuts a subtree" in _lib.lib().cbm_b200_last_error()
    # a tree with a repeated child is not a tree
    mc = c.mst_col.numpy().copy()
    mc[0] = mc[1]
    rc, _ = _schedule(c, mst_col=mc)
    assert rc == 3
    # labels that collide
    perm = np.arange(n)
    perm[1] = 0
    rc, _ = _schedule(c, perm=perm, n_labels=n)
    assert rc == 1
