"""Host-side checks of ``cbm4gnn_b200.cbm_mkl_cpp`` (the drop-in for the reference's native
module) that need no GPU: the builders' output layout, consumed by the reference's own compute
code and by the reference's own Python class."""
import contextlib
import io
import os
import sys

import numpy as np
import pytest
import torch

from cbm4gnn_b200 import cbm_mkl_cpp as shim
from cbm4gnn_b200 import graphs
from oracle import build_ref, reference

needs_ref = pytest.mark.skipif(not reference.ref_available(), reason="oracle/_ref has not been built")


def _sorted_edges(ei):
    order = np.lexsort((ei[1], ei[0]))
    return torch.from_numpy(np.ascontiguousarray(ei[:, order])).to(torch.int32)


def test_the_thirteen_names_are_there():
    names = ["from_coo_int32_t_v1_", "from_coo_int32_t_v2_", "seq_s_spmm_update_csr_int32", "seq_s_update_csr_int32",
             "seq_s_spmm_csr_int32", "omp_s_spmm_update_csr_int32", "omp_s_update_avx_int32", "omp_s_update_csr_int32",
             "omp_s_spmm_csr_int32", "omp_s_fused_spmm_update_csr_int32", "omp_s_fused_update_csr_int32",
             "seq_s_fused_spmm_update_csr_int32", "seq_s_fused_update_csr_int32"]  # cbm/cbm_extensions.cpp:1757-1771
    assert sorted(names) == sorted(shim.__all__)
    for n in names:
        assert callable(getattr(shim, n))


@needs_ref
@pytest.mark.parametrize("alpha", [0, 3])
def test_reference_compute_code_consumes_the_librarys_structure(alpha):
    """Builder output of the drop-in module, in the reference's five-tensor layout, multiplied by
    the reference's own compiled product: must give A @ X exactly (integer features)."""
    ref = reference.ref_module()
    e = _sorted_edges(graphs.make_graph("c1", scale=0.2))
    n = int(e.max()) + 1
    mst_row, mst_col, d_row, d_col, d_val = shim.from_coo_int32_t_v1_(e[0].contiguous(), e[1].contiguous(),
                                                                      torch.ones(e.shape[1]), n, n, alpha)
    assert mst_row.dtype == torch.int32 and mst_row.numel() == n + 2 and mst_col.numel() == n
    assert d_row.dtype == torch.int32 and d_col.dtype == torch.int32 and d_val.dtype == torch.float32
    csr = torch.sparse_coo_tensor(torch.stack((d_row, d_col)).long(), d_val, size=(n, n)).coalesce().to_sparse_csr()
    x = torch.randint(0, 10, (n, 24), generator=torch.Generator().manual_seed(3)).float()
    y = torch.zeros_like(x)
    ref.omp_s_spmm_update_csr_int32(csr.crow_indices()[:-1].to(torch.int32), csr.crow_indices()[1:].to(torch.int32),
                                    csr.col_indices().to(torch.int32), csr.values(), x, mst_row, mst_col, y)
    want = torch.sparse_coo_tensor(e.long(), torch.ones(e.shape[1]), size=(n, n)) @ x
    np.testing.assert_array_equal(y.numpy(), want.numpy())


@pytest.mark.skipif(build_ref.reference_source() is None, reason="needs the reference checkout")
@pytest.mark.parametrize("normalized", [False, True])
def test_reference_python_class_builds_on_the_drop_in_module(normalized):
    """The reference's unmodified cbm/cbm.py with ``cbm.cbm_mkl_cpp`` replaced by the drop-in
    module: construction, CSR conversion and its own ``check_format`` validator."""
    ref_dir = build_ref.DEFAULT_REFERENCE
    saved = {k: sys.modules.get(k) for k in ("cbm", "cbm.cbm", "cbm.cbm_mkl_cpp")}
    sys.path.insert(0, ref_dir)
    try:
        for k in saved:
            sys.modules.pop(k, None)
        import cbm
        sys.modules["cbm.cbm_mkl_cpp"] = shim
        cbm.cbm_mkl_cpp = shim
        from cbm.cbm import cbm_matrix as ref_cbm_matrix
        e = _sorted_edges(graphs.erdos_renyi(40, 0.3, 11))
        if normalized:
            n = int(e.max()) + 1
            loops = torch.arange(n, dtype=torch.int32)
            e = _sorted_edges(torch.cat([e, torch.stack([loops, loops])], dim=1).numpy())
        with contextlib.redirect_stdout(io.StringIO()):
            c = ref_cbm_matrix(e, torch.ones(e.shape[1]), alpha=2, normalized=normalized)
            c.check_format(e)
        assert c.mst_row.dtype == torch.int32 and c.deltas.layout == torch.sparse_csr
    finally:
        sys.path.remove(ref_dir)
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v
