"""Parity of the CUDA products with the CPU restatement, the fixtures and dense / sparse A @ X.

Every product here goes through the C ABI of libcbm_b200.so (``cbm_matrix`` methods are thin ctypes
calls).  Tolerance for floating-point inputs: atol = rtol = 1e-4 (fp32), the reference's own figure
(tests/test_matmul_correctness.py:43); integer-valued inputs must match bit for bit.
"""
import ctypes

import numpy as np
import pytest
import torch

from cbm4gnn_b200 import _lib, graphs
from cbm4gnn_b200.cbm import cbm_matrix, _Plan
from oracle import cbm_oracle as orc
from conftest import golden_case
from helpers import dense_product, sparse_product, with_self_loops

pytestmark = pytest.mark.gpu
TOL = dict(atol=1e-4, rtol=1e-4)


def _cbm(ei, alpha=0, normalized=False):
    e = torch.from_numpy(np.ascontiguousarray(ei)).to(torch.int32)
    return cbm_matrix(e, torch.ones(e.shape[1]), alpha=alpha, normalized=normalized)


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _oracle(c, x, parallel=True):
    mr, mc = c.mst_row.numpy(), c.mst_col.numpy()
    if c.normalized:
        return orc.fused_spmm_update(mr, mc, c._crow, c._dcol, c._dval, c.col_multiplier.numpy(), x, parallel)
    return orc.spmm_update(mr, mc, c._crow, c._dcol, c._dval, x, parallel)


@pytest.mark.parametrize("k", range(5))
@pytest.mark.parametrize("alpha", [0, 2, 3])
def test_golden_unnormalized_bit_exact(golden, k, alpha):
    ei, x, y, _ = golden_case(golden, k)
    c = _cbm(ei, alpha)
    xd = _dev(x)
    out = torch.full_like(xd, float("nan"))
    c.omp_mkl_csr_spmm_update(xd, out)
    np.testing.assert_array_equal(out.cpu().numpy(), y)
    out2 = torch.full_like(xd, float("nan"))
    c.seq_mkl_csr_spmm_update(xd, out2)
    assert torch.equal(out, out2)
    # two-step form of cbm/cbm.py:255-265
    np.testing.assert_array_equal(c.seq_torch_csr_matmul(xd).cpu().numpy(), y)
    np.testing.assert_array_equal(c.omp_torch_csr_matmul(xd).cpu().numpy(), y)
    c.plan().status()


@pytest.mark.parametrize("k", range(5))
def test_golden_normalized(golden, k):
    ei, x, _, y_norm = golden_case(golden, k)
    c = _cbm(with_self_loops(ei), 2, normalized=True)
    xd = _dev(x)
    out = torch.empty_like(xd)
    c.omp_mkl_csr_fused_spmm_update(xd, out)
    np.testing.assert_allclose(out.cpu().numpy(), y_norm, **TOL)
    np.testing.assert_allclose(c.omp_torch_csr_fused_matmul(xd).cpu().numpy(), y_norm, **TOL)
    np.testing.assert_allclose(out.cpu().numpy(), _oracle(c, x), **TOL)


def test_host_tensors_are_staged_through_the_gpu(golden):
    ei, x, y, y_norm = golden_case(golden, 0)
    c = _cbm(ei, 2)
    out = torch.empty((c.num_rows, x.shape[1]))
    c.omp_mkl_csr_spmm_update(torch.from_numpy(x), out)
    np.testing.assert_array_equal(out.numpy(), y)
    np.testing.assert_array_equal(c.seq_torch_csr_matmul(torch.from_numpy(x)).numpy(), y)
    cn = _cbm(with_self_loops(ei), 2, normalized=True)
    outn = torch.empty((c.num_rows, x.shape[1]))
    cn.seq_mkl_csr_fused_spmm_update(torch.from_numpy(x), outn)
    np.testing.assert_allclose(outn.numpy(), y_norm, **TOL)


@pytest.fixture(scope="module")
def c1():
    ei = graphs.make_graph("c1")
    return ei, _cbm(ei, 0)


def test_config1_full(c1):
    """N = 4096 copy-model graph, alpha = 0, unnormalized, F = 500, X uniform[0,1): against dense
    A @ X and against both CPU paths of the restatement."""
    ei, c = c1
    n = c.num_rows
    x = graphs.make_features("c1", n)
    out = torch.empty((n, 500), device="cuda")
    c.omp_mkl_csr_spmm_update(_dev(x), out)
    got = out.cpu().numpy()
    np.testing.assert_allclose(got, dense_product(ei, x, False), **TOL)
    np.testing.assert_allclose(got, _oracle(c, x, parallel=False), **TOL)
    np.testing.assert_allclose(got, _oracle(c, x, parallel=True), **TOL)
    c.plan().status()


@pytest.mark.parametrize("f", [1, 3, 4, 31, 47, 64, 100, 128, 132, 250, 256, 500, 516, 1024, 1100])
def test_operand_widths(c1, f):
    ei, c = c1
    n = c.num_rows
    rng = np.random.default_rng(f)
    x = rng.integers(-4, 5, size=(n, f)).astype(np.float32)  # exact in fp32
    want = sparse_product(ei, x, False).astype(np.float32)
    out = torch.empty((n, f), device="cuda")
    c.omp_mkl_csr_spmm_update(_dev(x), out)
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    d = torch.empty((n, f), device="cuda")
    c.omp_mkl_csr_spmm(_dev(x), d)
    np.testing.assert_array_equal(d.cpu().numpy(), orc.csr_spmm(c._crow, c._dcol, c._dval, x))
    c.omp_mkl_csr_update(d)
    np.testing.assert_array_equal(d.cpu().numpy(), want)


def test_strided_operands(c1):
    ei, c = c1
    n = c.num_rows
    rng = np.random.default_rng(1)
    for f, ld in ((64, 80), (30, 33), (128, 500)):
        xb = torch.zeros((n, ld), device="cuda")
        yb = torch.full((n, ld), -7.0, device="cuda")
        x = rng.integers(-4, 5, size=(n, f)).astype(np.float32)
        xb[:, :f] = _dev(x)
        c.omp_mkl_csr_spmm_update(xb[:, :f], yb[:, :f])
        np.testing.assert_array_equal(yb[:, :f].cpu().numpy(), sparse_product(ei, x, False).astype(np.float32))
        assert torch.all(yb[:, f:] == -7.0)  # nothing outside the view is touched


def test_config2_scaled_normalized():
    """Copy model p = 0.7, 5 random links, alpha = 8, D^-1/2 (A+I) D^-1/2, X ~ N(0,1)."""
    ei = with_self_loops(graphs.make_graph("c2", scale=0.1))
    c = _cbm(ei, 8, normalized=True)
    n = c.num_rows
    x = graphs.make_features("c2", n, f=500)
    out = torch.empty((n, 500), device="cuda")
    c.omp_mkl_csr_fused_spmm_update(_dev(x), out)
    got = out.cpu().numpy()
    np.testing.assert_allclose(got, sparse_product(ei, x, True), **TOL)
    np.testing.assert_allclose(got, _oracle(c, x), **TOL)
    # the weights of the plain-CSR comparison matrix (gnns/utility.py:25-33) give the same product
    from cbm4gnn_b200.utility import normalize_edge_index
    w = normalize_edge_index(torch.from_numpy(ei)).cuda()
    a = torch.sparse_coo_tensor(torch.from_numpy(ei).cuda(), w, (n, n)).to_sparse_csr()
    np.testing.assert_allclose(got, (a @ _dev(x)).cpu().numpy(), **TOL)
    # update-only form on the delta product
    d = torch.empty_like(out)
    c.seq_mkl_csr_spmm(_dev(x), d)
    c.seq_mkl_csr_fused_update(d)
    np.testing.assert_allclose(d.cpu().numpy(), got, **TOL)


def test_alpha_sweep_high_similarity():
    """Small stand-in for the high-similarity configuration: alpha in {0, 4, 16, 64}."""
    ei = with_self_loops(graphs.copy_model(3000, 0.95, 20, 77))
    n = int(ei.max()) + 1
    x = (np.random.default_rng(5).random((n, 128), dtype=np.float32) * 2 - 1).astype(np.float32)
    want = sparse_product(ei, x, True)
    prev = None
    for alpha in (0, 4, 16, 64):
        c = _cbm(ei, alpha, normalized=True)
        out = torch.empty((n, 128), device="cuda")
        c.omp_mkl_csr_fused_spmm_update(_dev(x), out)
        np.testing.assert_allclose(out.cpu().numpy(), want, **TOL)
        if prev is not None:
            assert c.build_info["n_delta"] >= prev  # a larger alpha never compresses more
        prev = c.build_info["n_delta"]


def test_deep_chain_and_repeated_calls():
    """Nested rows r_i = {0..i} give a tree that is one chain of depth n: every row waits for the
    row before it.  Also exercises repeated launches on one plan and changing widths."""
    n = 1500
    rows = np.repeat(np.arange(n), np.arange(1, n + 1))
    cols = np.concatenate([np.arange(i + 1) for i in range(n)])
    ei = np.stack([rows, cols])
    c = _cbm(ei, 0)
    assert c.build_info["depth"] == n and c.build_info["n_delta"] == n
    for f in (8, 128, 500, 8):
        x = np.random.default_rng(f).integers(-3, 4, size=(n, f)).astype(np.float32)
        want = np.cumsum(x.astype(np.float64), axis=0).astype(np.float32)
        for _ in range(3):
            out = torch.empty((n, f), device="cuda")
            c.omp_mkl_csr_spmm_update(_dev(x), out)
            np.testing.assert_array_equal(out.cpu().numpy(), want)
    c.plan().status()


def test_csr_spmm_any_matrix():
    """Plain CSR product with arbitrary fp32 values (the MKL CSR baseline of the reference,
    cbm/cbm_extensions.cpp:1707-1755), 4-array form, device pointers."""
    rng = np.random.default_rng(9)
    ei = graphs.make_graph("c1", scale=0.5)
    n = int(ei.max()) + 1
    import scipy.sparse as sp
    val = rng.standard_normal(ei.shape[1]).astype(np.float32)
    a = sp.csr_matrix((val, (ei[0], ei[1])), shape=(n, n))
    crow, col = a.indptr.astype(np.int32), a.indices.astype(np.int32)
    L = _lib.lib()
    for f in (47, 128, 500):
        x = rng.standard_normal((n, f)).astype(np.float32)
        y = torch.empty((n, f), device="cuda")
        rb, re_, cd, vd, xd = _dev(crow[:-1]), _dev(crow[1:]), _dev(col), _dev(a.data), _dev(x)
        _lib.check(L.cbm_b200_csr_spmm(n, rb.data_ptr(), re_.data_ptr(), cd.data_ptr(), vd.data_ptr(),
                                       xd.data_ptr(), f, y.data_ptr(), f, f,
                                       torch.cuda.current_stream().cuda_stream))
        np.testing.assert_allclose(y.cpu().numpy(), orc.csr_spmm(crow, col, a.data, x), **TOL)


def test_sharded_plans_cover_the_product():
    """Two plans, each owning whole subtrees of the virtual root under a relabelling, together
    reproduce the full product (the unit of the multi-GPU split)."""
    from cbm4gnn_b200.sharding import partition_subtrees
    ei = with_self_loops(graphs.make_graph("c1"))
    c = _cbm(ei, 0, normalized=True)
    n = c.num_rows
    part = partition_subtrees(c, 2)
    x = graphs.make_features("c1", n, f=64)
    want = sparse_product(ei, x, True)
    xp = np.zeros((part.n_labels, 64), dtype=np.float32)
    xp[part.perm] = x            # the operand is indexed by label
    xd = _dev(xp)
    y_full = torch.zeros((part.n_labels, 64), device="cuda")
    for g in range(2):
        b, e = part.offsets(g)
        plan = _Plan(n, c.mst_row.numpy(), c.mst_col.numpy(), c._crow, c._dcol, c._dval,
                     c.col_multiplier.numpy(), 0, perm=part.perm, n_labels=part.n_labels, own_begin=b,
                     own_end=e)
        assert plan.n_rows == part.counts[g]
        y = y_full[b:e]
        _lib.check(_lib.lib().cbm_b200_fused_spmm_update(plan.handle, xd.data_ptr(), 64, y.data_ptr(), 64, 64,
                                                         torch.cuda.current_stream().cuda_stream))
        plan.status()
    np.testing.assert_allclose(y_full.cpu().numpy()[part.perm], want, **TOL)
    # an owned range that cuts a subtree is refused
    with pytest.raises(RuntimeError, match="cuts a subtree|owned"):
        ident = np.arange(n, dtype=np.int32)
        deep = int(np.nonzero(c._parent != n)[0][0])
        _Plan(n, c.mst_row.numpy(), c.mst_col.numpy(), c._crow, c._dcol, c._dval, c.col_multiplier.numpy(), 0,
              perm=ident, n_labels=n, own_begin=deep, own_end=deep + 1)


def test_argument_errors(c1):
    _, c = c1
    n = c.num_rows
    x = torch.ones((n, 8), device="cuda")
    with pytest.raises(RuntimeError, match="kFloat32"):
        c.omp_mkl_csr_spmm_update(x.double(), torch.empty((n, 8), device="cuda"))
    with pytest.raises(RuntimeError, match="shape"):
        c.omp_mkl_csr_spmm_update(x, torch.empty((n, 9), device="cuda"))
    with pytest.raises(RuntimeError, match="col_multiplier"):
        c.omp_mkl_csr_fused_spmm_update(x, torch.empty_like(x))
    with pytest.raises(RuntimeError, match="alias"):
        c.omp_mkl_csr_spmm_update(x, x)
    p = c.plan()
    bad = ctypes.c_void_p(0)
    assert _lib.lib().cbm_b200_plan_create(n, c.mst_row.numpy().ctypes.data, c.mst_col.numpy().ctypes.data,
                                           c._crow.ctypes.data, c._dcol.ctypes.data, c._dval.ctypes.data, None,
                                           None, 0, 0, n, 99, ctypes.byref(bad)) != 0
    # a tree with a cycle is refused
    mr = c.mst_row.numpy().copy()
    mc = c.mst_col.numpy().copy()
    mc[0] = mc[1]
    assert _lib.lib().cbm_b200_plan_create(n, mr.ctypes.data, mc.ctypes.data, c._crow.ctypes.data,
                                           c._dcol.ctypes.data, c._dval.ctypes.data, None, None, 0, 0, n, 0,
                                           ctypes.byref(bad)) == 3
    p.status()


@pytest.fixture(scope="module")
def c2_full():
    ei = with_self_loops(graphs.make_graph("c2"))
    return ei, _cbm(ei, 8, normalized=True)


def test_config2_full_size_properties(c2_full):
    """At the benchmark's full size (N = 100 000, F = 500) the CPU restatement is too slow for a
    unit test, so parity is checked on a row sample against float64 CSR and through linearity:
    A(2x - 3z) == 2 A x - 3 A z."""
    ei, c = c2_full
    n = c.num_rows
    x = graphs.make_features("c2", n)
    z = graphs.make_features("c2", n, seed_offset=2000)
    xd, zd = _dev(x), _dev(z)
    yx, yz, yc = (torch.empty((n, 500), device="cuda") for _ in range(3))
    c.omp_mkl_csr_fused_spmm_update(xd, yx)
    c.omp_mkl_csr_fused_spmm_update(zd, yz)
    c.omp_mkl_csr_fused_spmm_update(2 * xd - 3 * zd, yc)
    torch.testing.assert_close(yc, 2 * yx - 3 * yz, atol=1e-3, rtol=1e-4)
    rows = np.random.default_rng(0).choice(n, 2000, replace=False)
    import scipy.sparse as sp
    a = sp.csr_matrix((np.ones(ei.shape[1]), (ei[0], ei[1])), shape=(n, n))
    s = np.asarray(a.sum(1)).ravel() ** -0.5
    want = (sp.diags(s[rows]) @ a[rows] @ sp.diags(s)) @ x.astype(np.float64)
    np.testing.assert_allclose(yx[torch.from_numpy(rows).cuda()].cpu().numpy(), want, **TOL)
    c.plan().status()


def test_bulk_copy_form_matches_register_form(c1):
    """The opt-in kernel form that stages operand rows in shared memory with bulk asynchronous
    copies performs the same arithmetic in the same order: results must be identical."""
    ei, c = c1
    n = c.num_rows
    p = c.plan()
    L = _lib.lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    try:
        for f in (500, 256, 64, 4):
            # integer-valued operand: every summation order gives the same floats
            x = torch.randint(-4, 5, (n, f), device="cuda").float()
            ya, yb, da_, db_ = (torch.full((n, f), float("nan"), device="cuda") for _ in range(4))
            p.tune(form=0)
            _lib.check(L.cbm_b200_spmm_update(p.handle, x.data_ptr(), f, ya.data_ptr(), f, f, st))
            _lib.check(L.cbm_b200_delta_spmm(p.handle, x.data_ptr(), f, da_.data_ptr(), f, f, st))
            p.tune(form=1)
            _lib.check(L.cbm_b200_spmm_update(p.handle, x.data_ptr(), f, yb.data_ptr(), f, f, st))
            _lib.check(L.cbm_b200_delta_spmm(p.handle, x.data_ptr(), f, db_.data_ptr(), f, f, st))
            p.status()
            assert torch.equal(ya, yb) and torch.equal(da_, db_)
    finally:
        p.tune(form=0)


def test_host_operands_pinned_and_pageable_agree(c1):
    """Page-locked host operands travel through copy kernels, pageable ones through the runtime's
    copies; both must give the device-resident result exactly."""
    ei, c = c1
    n = c.num_rows
    for f in (500, 130, 64):
        x = torch.randn((n, f))
        want = torch.empty((n, f), device="cuda")
        c.omp_mkl_csr_spmm_update(x.cuda(), want)
        got_pageable = torch.empty((n, f))
        c.omp_mkl_csr_spmm_update(x, got_pageable)
        got_pinned = torch.empty((n, f)).pin_memory()
        c.omp_mkl_csr_spmm_update(x.pin_memory(), got_pinned)
        assert torch.equal(got_pageable, want.cpu()) and torch.equal(got_pinned, want.cpu())


def test_bounded_wait_reports_timeout_and_context_survives(c1):
    """A wait for a flag nothing sets must end by itself with the timeout status (50 ms limit);
    afterwards the same context still computes correct products."""
    L = _lib.lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.cbm_b200_selftest_wait(torch.cuda.current_device(), 50, st) == 4
    assert b"ran out as it should" in L.cbm_b200_last_error()
    assert L.cbm_b200_selftest_wait(torch.cuda.current_device(), 0, st) == 1
    ei, c = c1
    x = torch.randint(-3, 4, (c.num_rows, 8), device="cuda").float()
    y = torch.empty_like(x)
    c.omp_mkl_csr_spmm_update(x, y)
    np.testing.assert_array_equal(y.cpu().numpy(), sparse_product(ei, x.cpu().numpy(), False).astype(np.float32))
    c.plan().status()


def test_structure_in_reference_layout_is_consumed_unmodified(golden):
    """A structure that already exists as (mst_row, mst_col, delta CSR, multiplier) arrays — what
    the reference's own builder returns — runs without going through this package's builder.
    Here the arrays come from the independent restatement, whose tree differs from the product
    builder's wherever optimal trees tie."""
    ei, x, y, y_norm = golden_case(golden, 3)
    s = orc.build_structure(ei, 1)
    c = cbm_matrix.from_arrays(s["mst_row"], s["mst_col"], s["crow"], s["col"], s["val"])
    out = torch.empty((s["n"], x.shape[1]), device="cuda")
    c.omp_mkl_csr_spmm_update(_dev(x), out)
    np.testing.assert_array_equal(out.cpu().numpy(), y)
    eil = with_self_loops(ei)
    mult = orc.row_multiplier(eil, s["n"])
    sn = orc.build_structure(eil, 2, col_mul=mult)
    cn = cbm_matrix.from_arrays(sn["mst_row"], sn["mst_col"], sn["crow"], sn["col"], sn["val"], col_multiplier=mult)
    outn = torch.empty_like(out)
    cn.omp_mkl_csr_fused_spmm_update(_dev(x), outn)
    np.testing.assert_allclose(outn.cpu().numpy(), y_norm, **TOL)
    cn.check_format(torch.from_numpy(eil))


def test_giant_row_collects_hundreds_of_parked_shares():
    """A hub row with 40 000 delta entries is cut into 313 segments; the finishing item must wait
    for and add 312 parked shares (done 32 flags and 8 shares at a time)."""
    n = 40001
    hub = np.zeros(n - 1, dtype=np.int64)
    leaf = np.arange(1, n, dtype=np.int64)
    ei = np.stack([np.concatenate([hub, leaf]), np.concatenate([leaf, hub])])
    # alpha above every row length: no compression is attempted (on a star the candidate search
    # would visit all 40 000^2 leaf pairs, as the reference's A*A^T does), every row hangs off the
    # virtual root and the hub row keeps all its entries
    c = _cbm(ei, 100000)
    assert int(np.diff(c._crow).max()) == n - 1
    for f in (64, 500):
        x = np.random.default_rng(f).integers(-2, 3, size=(n, f)).astype(np.float32)
        out = torch.empty((n, f), device="cuda")
        c.omp_mkl_csr_spmm_update(_dev(x), out)
        np.testing.assert_array_equal(out.cpu().numpy(), sparse_product(ei, x, False).astype(np.float32))
    c.plan().status()


def test_alpha_search_measures_on_the_gpu():
    """Every alpha of the sweep is timed on the GPU; the structure the search settles on must
    multiply correctly (against float64 CSR) and the table must agree with the builder's figures."""
    from cbm4gnn_b200.alpha_search import product_bytes, search_alpha
    ei_np = with_self_loops(graphs.copy_model(3000, 0.95, 8, 5))
    ei = torch.from_numpy(ei_np)
    best, table = search_alpha(ei, f=64, alphas=(0, 4, 64), normalized=True, iters=5)
    assert [r["alpha"] for r in table] == [0, 4, 64]
    assert best == min(table, key=lambda r: (r["ms"], r["alpha"]))["alpha"]
    assert all(0.001 < r["ms"] < 50 for r in table)
    n = int(ei.max()) + 1
    for r in table:
        c = _cbm(ei_np, r["alpha"], normalized=True)
        assert c.build_info["n_delta"] == r["n_delta"] and c.build_info["depth"] == r["depth"]
        assert r["bytes"] == product_bytes(n, r["n_delta"], r["n_root_children"], 64)
    assert table[0]["n_delta"] <= table[1]["n_delta"] <= table[2]["n_delta"]
    x = np.random.default_rng(3).standard_normal((n, 64)).astype(np.float32)
    c = _cbm(ei_np, best, normalized=True)
    y = torch.empty((n, 64), device="cuda")
    c.omp_mkl_csr_fused_spmm_update(_dev(x), y)
    np.testing.assert_allclose(y.cpu().numpy(), sparse_product(ei_np, x, True), **TOL)


def test_csr_plan_balances_long_rows_and_matches_the_array_form():
    """Plain CSR through a plan (every row a child of the virtual root, long rows cut into
    segments) against the array form and float64, on a matrix with one 30 000-entry row,
    rectangular, arbitrary values."""
    from cbm4gnn_b200.cbm import csr_matrix_plan
    import scipy.sparse as sp
    rng = np.random.default_rng(21)
    n_rows, n_cols = 5000, 30000
    dense_row = np.stack([np.zeros(n_cols, dtype=np.int64), np.arange(n_cols)])
    rest = np.stack([rng.integers(1, n_rows, 60000), rng.integers(0, n_cols, 60000)])
    ij = np.concatenate([dense_row, rest], axis=1)
    a = sp.csr_matrix((rng.standard_normal(ij.shape[1]).astype(np.float32), (ij[0], ij[1])), shape=(n_rows, n_cols))
    a.sum_duplicates()
    a.sort_indices()
    plan = csr_matrix_plan(a.indptr, a.indices, a.data, n_cols)
    for f in (128, 47):
        x = rng.standard_normal((n_cols, f)).astype(np.float32)
        y = plan.matmul(_dev(x))
        plan.status()
        want = a.astype(np.float64) @ x.astype(np.float64)
        np.testing.assert_allclose(y.cpu().numpy(), want, atol=2e-3, rtol=1e-4)  # 30 000-term fp32 sums
        np.testing.assert_allclose(y.cpu().numpy()[1:], want[1:], **TOL)
    with pytest.raises(RuntimeError, match="shape mismatch"):
        plan.matmul(torch.zeros((n_cols + 1, 8), device="cuda"))


def test_broadcast_epilogue_writes_every_destination(c1):
    """The multi-GPU form of the product on one GPU: finished rows go to y and, after the ReLU,
    to further buffers with y's layout (on several GPUs these are the peers' gathered buffers)."""
    ei, _ = c1
    eil = with_self_loops(ei)
    c = _cbm(eil, 2, normalized=True)
    n = c.num_rows
    L = _lib.lib()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for f, ld in ((500, 500), (64, 64), (47, 47), (128, 160)):
        x = torch.randn((n, f), device="cuda")
        want = torch.empty((n, f), device="cuda")
        c.omp_mkl_csr_fused_spmm_update(x, want)
        y = torch.full((n, ld), float("nan"), device="cuda")
        dst = [torch.full((n, ld), float("nan"), device="cuda") for _ in range(3)]
        arr = (ctypes.c_void_p * 3)(*[d.data_ptr() for d in dst])
        _lib.check(L.cbm_b200_spmm_update_bcast(c.plan().handle, x.data_ptr(), f, y.data_ptr(), ld, f, 1, 1, 3, arr, st))
        c.plan().status()
        assert torch.equal(y[:, :f], want)                     # the tree's own copy: no ReLU
        for d in dst:
            assert torch.equal(d[:, :f], want.relu())
            assert torch.isnan(d[:, f:]).all()                 # nothing outside the rows' width
    assert L.cbm_b200_spmm_update_bcast(c.plan().handle, x.data_ptr(), f, y.data_ptr(), ld, f, 1, 0, 9, arr, st) == 1


def test_host_operands_with_ragged_width(c1):
    """Host tensors whose width is not a multiple of 4 (the 47-wide output layer of the fifth
    configuration): the staged product equals the device-resident one exactly."""
    ei, c = c1
    n = c.num_rows
    for f in (47, 131, 5, 3):
        # integer-valued operand: the staged path cuts the width into a 128-bit part and a scalar
        # tail, which sum in another order than the device-resident path; integers make both exact
        x = torch.randint(-4, 5, (n, f)).float()
        want = torch.empty((n, f), device="cuda")
        c.omp_mkl_csr_spmm_update(x.cuda(), want)
        got = torch.empty((n, f))
        c.omp_mkl_csr_spmm_update(x, got)
        assert torch.equal(got, want.cpu())
        np.testing.assert_array_equal(got.numpy(), sparse_product(ei, x.numpy(), False).astype(np.float32))
        xr = torch.randn((n, f))
        c.omp_mkl_csr_spmm_update(xr, got)
        np.testing.assert_allclose(got.numpy(), sparse_product(ei, xr.numpy(), False), **TOL)


def test_l2_probe_reports_a_plausible_rate():
    r = _lib.lib().cbm_b200_probe_l2_read_gbps(torch.cuda.current_device())
    assert 2000.0 < r < 60000.0
