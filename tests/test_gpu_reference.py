"""CUDA products against the reference itself.

Three layers, all through the C ABI of libcbm_b200.so:
* the committed fixtures the reference produced (tests/golden/cbm_reference.npz): the CUDA engine
  consumes the reference's own structure arrays unmodified and must reproduce every product method
  of cbm/cbm.py:144-275;
* ``oracle/_ref`` (the reference's unmodified native source, prebuilt) run live on the host beside
  the GPU at the sizes of the first two benchmark configurations;
* ``cbm4gnn_b200.cbm_mkl_cpp``, the drop-in for the reference's native module, called with the
  reference's argument lists next to ``oracle/_ref`` called with the same arguments.

Tolerance atol = rtol = 1e-4 (tests/test_matmul_correctness.py:43); integer-valued inputs bit for bit.
"""
import numpy as np
import pytest
import torch

from cbm4gnn_b200 import cbm_mkl_cpp as shim
from cbm4gnn_b200 import graphs
from cbm4gnn_b200.cbm import cbm_matrix
from oracle import reference
from helpers import with_self_loops

pytestmark = pytest.mark.gpu
TOL = dict(atol=1e-4, rtol=1e-4)
NAMES = ["er25a", "er25b", "er40", "er64", "copy300"]
needs_ref = pytest.mark.skipif(not reference.ref_available(), reason="oracle/_ref has not been built")


def _close(got, want, exact):
    got = got.cpu().numpy() if isinstance(got, torch.Tensor) else got
    if exact:
        np.testing.assert_array_equal(got, want)
    else:
        np.testing.assert_allclose(got, want, **TOL)


@pytest.mark.parametrize("name", NAMES)
def test_reference_structure_and_outputs_plain(ref_golden, name):
    g = ref_golden.case(name, False)
    c = cbm_matrix.from_arrays(g["mst_row"], g["mst_col"], g["crow"], g["col"], g["val"])
    exact = name.startswith("er25")  # integer-valued features
    xd = torch.from_numpy(g["x"]).cuda()
    for m in ("seq_mkl_csr_spmm_update", "omp_mkl_csr_spmm_update"):
        y = torch.full_like(xd, float("nan"))
        getattr(c, m)(xd, y)
        _close(y, g[m], exact)
    for m in ("seq_mkl_csr_spmm", "omp_mkl_csr_spmm"):
        y = torch.full_like(xd, float("nan"))
        getattr(c, m)(xd, y)
        _close(y, g[m], exact)
    for m in ("seq_mkl_csr_update", "omp_mkl_csr_update", "omp_avx_csr_update"):
        if m in g:
            y = torch.from_numpy(g["delta_x"].copy()).cuda()
            getattr(c, m)(y)
            _close(y, g[m], exact)
    for m in ("seq_torch_csr_matmul", "omp_torch_csr_matmul"):
        _close(getattr(c, m)(xd), g[m], exact)
    c.plan().status()


@pytest.mark.parametrize("name", NAMES)
def test_reference_structure_and_outputs_normalized(ref_golden, name):
    g = ref_golden.case(name, True)
    c = cbm_matrix.from_arrays(g["mst_row"], g["mst_col"], g["crow"], g["col"], g["val"], g["col_multiplier"])
    xd = torch.from_numpy(g["x"]).cuda()
    for m in ("seq_mkl_csr_fused_spmm_update", "omp_mkl_csr_fused_spmm_update"):
        y = torch.full_like(xd, float("nan"))
        getattr(c, m)(xd, y)
        _close(y, g[m], False)
    for m in ("seq_mkl_csr_fused_update", "omp_mkl_csr_fused_update"):
        y = torch.from_numpy(g["delta_x"].copy()).cuda()
        getattr(c, m)(y)
        _close(y, g[m], False)
    _close(c.seq_torch_csr_fused_matmul(xd), g["seq_torch_csr_fused_matmul"], False)
    _close(c.omp_torch_csr_fused_matmul(xd), g["seq_torch_csr_fused_matmul"], False)
    # host tensors through the same methods, as every caller of the reference passes them
    y = torch.empty(g["x"].shape)
    c.omp_mkl_csr_fused_spmm_update(torch.from_numpy(g["x"]), y)
    _close(y, g["omp_mkl_csr_fused_spmm_update"], False)
    c.plan().status()


def _ref_args(c):
    crow = torch.from_numpy(c._crow)
    return crow[:-1].contiguous(), crow[1:].contiguous(), torch.from_numpy(c._dcol), torch.from_numpy(c._dval)


@needs_ref
def test_config1_full_size_against_compiled_reference():
    """N = 4096, alpha = 0, unnormalized, F = 500: the configuration the reference runs as it is."""
    ref = reference.ref_module()
    ei = graphs.make_graph("c1")
    e = torch.from_numpy(ei).to(torch.int32)
    c = cbm_matrix(e, torch.ones(e.shape[1]), alpha=0)
    x = torch.from_numpy(graphs.make_features("c1", c.num_rows))
    rb, re_, col, val = _ref_args(c)
    want_seq, want_omp = torch.zeros_like(x), torch.zeros_like(x)
    ref.seq_s_spmm_update_csr_int32(rb, re_, col, val, x, c.mst_row, c.mst_col, want_seq)
    ref.omp_s_spmm_update_csr_int32(rb, re_, col, val, x, c.mst_row, c.mst_col, want_omp)
    y = torch.empty_like(x, device="cuda")
    c.omp_mkl_csr_spmm_update(x.cuda(), y)
    _close(y, want_seq.numpy(), False)
    _close(y, want_omp.numpy(), False)
    # integer features: every partial sum is exact in fp32, so the reference pins each bit
    xi = torch.randint(0, 10, x.shape, generator=torch.Generator().manual_seed(5)).float()
    want = torch.zeros_like(xi)
    ref.omp_s_spmm_update_csr_int32(rb, re_, col, val, xi, c.mst_row, c.mst_col, want)
    c.omp_mkl_csr_spmm_update(xi.cuda(), y)
    _close(y, want.numpy(), True)
    c.plan().status()


@needs_ref
def test_config2_full_size_against_compiled_reference():
    """N = 100 000, alpha = 8, normalized with self loops, F = 500: the benchmark's workload, every
    output element against the reference's OpenMP + oneMKL path run on the host."""
    ref = reference.ref_module()
    ei = with_self_loops(graphs.make_graph("c2"))
    e = torch.from_numpy(ei).to(torch.int32)
    c = cbm_matrix(e, torch.ones(e.shape[1]), alpha=8, normalized=True)
    x = torch.from_numpy(graphs.make_features("c2", c.num_rows))
    rb, re_, col, val = _ref_args(c)
    want = torch.zeros_like(x)
    ref.omp_s_fused_spmm_update_csr_int32(rb, re_, col, val, x, c.mst_row, c.mst_col, c.col_multiplier, want)
    y = torch.empty_like(x, device="cuda")
    c.omp_mkl_csr_fused_spmm_update(x.cuda(), y)
    _close(y, want.numpy(), False)
    # update-only form on the reference's own delta product
    d = torch.zeros_like(x)
    ref.omp_s_spmm_csr_int32(rb, re_, col, val, x, d)
    dd = d.cuda()
    c.omp_mkl_csr_fused_update(dd)
    ref.omp_s_fused_update_csr_int32(c.mst_row, c.mst_col, c.col_multiplier, d)
    _close(dd, d.numpy(), False)
    c.plan().status()


@needs_ref
@pytest.mark.parametrize("normalized", [False, True])
def test_drop_in_module_beside_the_compiled_reference(normalized):
    """The same call, with the reference's argument list, into the drop-in module and into the
    reference's native module: 11 compute functions, CPU tensors as the reference's callers pass."""
    ref = reference.ref_module()
    ei = graphs.make_graph("c1", scale=0.25)
    if normalized:
        ei = with_self_loops(ei)
    order = np.lexsort((ei[1], ei[0]))
    e = torch.from_numpy(np.ascontiguousarray(ei[:, order])).to(torch.int32)
    n = int(e.max()) + 1
    ones = torch.ones(e.shape[1])
    if normalized:
        mul = torch.bincount(e[0].long(), minlength=n).float().pow(-0.5)
        mine = shim.from_coo_int32_t_v2_(e[0].contiguous(), e[1].contiguous(), ones, mul, n, n, 2)
        theirs = ref.from_coo_int32_t_v2_(e[0].contiguous(), e[1].contiguous(), ones, mul, n, n, 2)
    else:
        mine = shim.from_coo_int32_t_v1_(e[0].contiguous(), e[1].contiguous(), ones, n, n, 2)
        theirs = ref.from_coo_int32_t_v1_(e[0].contiguous(), e[1].contiguous(), ones, n, n, 2)
    assert [t.dtype for t in mine] == [t.dtype for t in theirs]
    assert [t.shape for t in mine] == [t.shape for t in theirs]  # same weight => same number of deltas
    # both structures, each through both modules
    x = torch.randint(-3, 4, (n, 64), generator=torch.Generator().manual_seed(1)).float()
    for mst_row, mst_col, d_row, d_col, d_val in (mine, theirs):
        csr = torch.sparse_coo_tensor(torch.stack((d_row, d_col)).long(), d_val, size=(n, n)).coalesce().to_sparse_csr()
        rb = csr.crow_indices()[:-1].to(torch.int32)
        re_ = csr.crow_indices()[1:].to(torch.int32)
        col, val = csr.col_indices().to(torch.int32), csr.values()
        for pre in ("seq", "omp"):
            def both(fn, *args_before_dst, inplace_src=None):
                outs = []
                for mod in (shim, ref):
                    dst = torch.zeros_like(x) if inplace_src is None else inplace_src.clone()
                    getattr(mod, fn)(*args_before_dst, dst)
                    outs.append(dst)
                return outs
            a, b = both(f"{pre}_s_spmm_csr_int32", rb, re_, col, val, x)
            _close(a, b.numpy(), not normalized)
            delta_x = b
            if normalized:
                a, b = both(f"{pre}_s_fused_spmm_update_csr_int32", rb, re_, col, val, x, mst_row, mst_col, mul)
                _close(a, b.numpy(), False)
                a, b = both(f"{pre}_s_fused_update_csr_int32", mst_row, mst_col, mul, inplace_src=delta_x)
                _close(a, b.numpy(), False)
            else:
                a, b = both(f"{pre}_s_spmm_update_csr_int32", rb, re_, col, val, x, mst_row, mst_col)
                _close(a, b.numpy(), True)
                a, b = both(f"{pre}_s_update_csr_int32", mst_row, mst_col, inplace_src=delta_x)
                _close(a, b.numpy(), True)
        if not normalized:
            a = delta_x.clone()
            shim.omp_s_update_avx_int32(mst_row, mst_col, a)
            b = delta_x.clone()
            ref.omp_s_update_avx_int32(mst_row, mst_col, b)  # width 64: the AVX loop's step bug does not bite
            _close(a, b.numpy(), True)


def test_drop_in_module_accepts_cuda_tensors():
    ei = graphs.make_graph("c1", scale=0.1)
    order = np.lexsort((ei[1], ei[0]))
    e = torch.from_numpy(np.ascontiguousarray(ei[:, order])).to(torch.int32)
    n = int(e.max()) + 1
    mst_row, mst_col, d_row, d_col, d_val = shim.from_coo_int32_t_v1_(e[0].contiguous(), e[1].contiguous(),
                                                                      torch.ones(e.shape[1]), n, n, 0)
    csr = torch.sparse_coo_tensor(torch.stack((d_row, d_col)).long(), d_val, size=(n, n)).coalesce().to_sparse_csr()
    rb, re_ = csr.crow_indices()[:-1].to(torch.int32), csr.crow_indices()[1:].to(torch.int32)
    x = torch.randint(0, 5, (n, 40)).float()
    y = torch.zeros((n, 40), device="cuda")
    shim.omp_s_spmm_update_csr_int32(rb, re_, csr.col_indices().to(torch.int32), csr.values(), x.cuda(), mst_row, mst_col, y)
    a = torch.sparse_coo_tensor(e.long(), torch.ones(e.shape[1]), size=(n, n)) @ x
    np.testing.assert_array_equal(y.cpu().numpy(), a.numpy())
    with pytest.raises(RuntimeError, match="NOT torch::kFloat32"):
        shim.omp_s_update_csr_int32(mst_row, mst_col, torch.zeros((n, 4), dtype=torch.float64, device="cuda"))
