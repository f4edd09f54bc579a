"""The allocation-free product entry point against the ordinary one.

``cbm_b200_spmm_update_static`` exists for callers that may not allocate device memory while they
run (all memory handed to their own pool, a stream capture in progress, a latency budget that an
allocation's device synchronisation would break).  It runs the same kernel as the ordinary entry
points but keeps its ready flags and partial sums in a fixed array inside the library, which is
shared between calls and keeps the previous call's contents.  The test therefore makes two calls in
a row, with different operands and a plan that has long rows (so partial sums are in play), and
requires each to reproduce the ordinary entry point exactly (both run the same arithmetic in the
same order) and to agree with an independent float64 CSR product of the same matrix.  The file name sorts last so that a run that stops at the first failure has already
exercised everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from cbm4gnn_b200 import _lib, graphs
from cbm4gnn_b200.cbm import cbm_matrix
from cbm4gnn_b200.utility import add_self_loops

pytestmark = pytest.mark.gpu


def _call(fn, plan, x, y, f, *extra):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(fn(plan.handle, x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), f, *extra, stream))


def test_static_scratch_product_matches_twice_in_a_row():
    L = _lib.lib()
    ei = add_self_loops(torch.from_numpy(graphs.make_graph("c1")))
    c = cbm_matrix(ei.to(torch.int32), torch.ones(ei.shape[1]), alpha=0, normalized=True)
    assert int(np.diff(c._crow).max()) > 192       # some rows are cut into segments
    plan = c.plan(torch.cuda.current_device())
    n = c.num_rows
    gen = torch.Generator(device="cuda").manual_seed(7)
    import scipy.sparse as sp
    e = ei.numpy()
    a64 = sp.csr_matrix((np.ones(e.shape[1]), (e[0], e[1])), shape=(n, n))
    s = np.asarray(a64.sum(1)).ravel() ** -0.5
    a64_norm = sp.diags(s) @ a64 @ sp.diags(s)
    for normalized, f in ((1, 500), (0, 64)):
        x = torch.randn((n, f), device="cuda", generator=gen)
        want = torch.empty((n, f), device="cuda")
        _call(L.cbm_b200_fused_spmm_update if normalized else L.cbm_b200_spmm_update, plan, x, want, f)
        got = torch.full((n, f), float("nan"), device="cuda")
        _call(L.cbm_b200_spmm_update_static, plan, x, got, f, normalized)
        plan.status()
        torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)
        assert torch.equal(got, want)
        # and both against an independent float64 CSR product of the same matrix
        # the plan carries the normalized structure (delta values +-s_col): without the row
        # scales of the fused form it computes A D^-1/2 x
        ref = a64_norm if normalized else a64 @ sp.diags(s)
        np.testing.assert_allclose(got.cpu().numpy(), ref @ x.cpu().numpy().astype(np.float64), atol=1e-4, rtol=1e-4)


def test_static_scratch_rejects_oversized_products():
    L = _lib.lib()
    # nested rows: row i holds columns 0..i, so one row alone has far more than 192 entries and
    # the operand is wide: the partial sums do not fit the fixed array
    n = 4000
    rows = np.repeat(np.arange(n), np.arange(1, n + 1))
    cols = np.concatenate([np.arange(i + 1) for i in range(n)])
    c = cbm_matrix(torch.from_numpy(np.stack([rows, cols])).to(torch.int32), torch.ones(rows.size), alpha=100000)
    plan = c.plan(torch.cuda.current_device())
    f = 1024
    x = torch.zeros((n, f), device="cuda")
    y = torch.zeros((n, f), device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.cbm_b200_spmm_update_static(plan.handle, x.data_ptr(), f, y.data_ptr(), f, f, 0, stream)
    assert rc == 1
    msg = L.cbm_b200_last_error().decode()
    assert "bytes of scratch" in msg and str(8 << 20) in msg
