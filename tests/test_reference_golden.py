"""The CPU restatement and the host builder against what the reference itself produced.

``tests/golden/cbm_reference.npz`` holds outputs of the reference's unmodified Python class and
native source (see tests/golden/make_golden_ref.py); where ``oracle/_ref`` is present the same
comparisons are repeated live against the compiled reference on larger inputs.  No GPU needed.
"""
import numpy as np
import pytest
import torch

from cbm4gnn_b200 import graphs
from cbm4gnn_b200.cbm import cbm_matrix
from oracle import cbm_oracle as orc
from oracle import reference

TOL = dict(atol=1e-4, rtol=1e-4)  # tests/test_matmul_correctness.py:43
NAMES = ["er25a", "er25b", "er40", "er64", "copy300"]


@pytest.mark.parametrize("name", NAMES)
def test_restated_updates_equal_the_reference_bit_for_bit(ref_golden, name):
    """Tree updates are plain fp32 adds / multiplies in a fixed order: the C restatement must
    reproduce the reference's compiled loops exactly, sequential and OpenMP forms alike."""
    g = ref_golden.case(name, False)
    for parallel, key in ((False, "seq_mkl_csr_update"), (True, "omp_mkl_csr_update")):
        got = orc.update(g["mst_row"], g["mst_col"], g["delta_x"].copy(), parallel)
        np.testing.assert_array_equal(got, g[key])
    if "omp_avx_csr_update" in g:
        np.testing.assert_array_equal(got, g["omp_avx_csr_update"])
    g = ref_golden.case(name, True)
    for parallel, key in ((False, "seq_mkl_csr_fused_update"), (True, "omp_mkl_csr_fused_update")):
        got = orc.fused_update(g["mst_row"], g["mst_col"], g["col_multiplier"], g["delta_x"].copy(), parallel)
        np.testing.assert_array_equal(got, g[key])


@pytest.mark.parametrize("name", NAMES)
def test_restated_products_match_the_reference(ref_golden, name):
    g = ref_golden.case(name, False)
    for parallel in (False, True):
        got = orc.spmm_update(g["mst_row"], g["mst_col"], g["crow"], g["col"], g["val"], g["x"], parallel)
        for key in ("seq_mkl_csr_spmm_update", "omp_mkl_csr_spmm_update", "seq_torch_csr_matmul", "omp_torch_csr_matmul"):
            np.testing.assert_allclose(got, g[key], **TOL)
        np.testing.assert_allclose(orc.csr_spmm(g["crow"], g["col"], g["val"], g["x"], parallel), g["seq_mkl_csr_spmm"], **TOL)
    g = ref_golden.case(name, True)
    for parallel in (False, True):
        got = orc.fused_spmm_update(g["mst_row"], g["mst_col"], g["crow"], g["col"], g["val"], g["col_multiplier"],
                                    g["x"], parallel)
        for key in ("seq_mkl_csr_fused_spmm_update", "omp_mkl_csr_fused_spmm_update", "seq_torch_csr_fused_matmul"):
            np.testing.assert_allclose(got, g[key], **TOL)


@pytest.mark.parametrize("name", NAMES[:2])
def test_integer_features_pin_the_plain_product_exactly(ref_golden, name):
    g = ref_golden.case(name, False)
    got = orc.spmm_update(g["mst_row"], g["mst_col"], g["crow"], g["col"], g["val"], g["x"], True)
    np.testing.assert_array_equal(got, g["omp_mkl_csr_spmm_update"])


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("normalized", [False, True])
def test_host_builder_against_the_reference_structure(ref_golden, name, normalized):
    """Same input, the library's builder against cbm_init_v1_/v2_ of the reference: equal number
    of delta entries (= weight of a minimum-cost arborescence, unique even where the tree is not),
    bit-equal multiplier, and the reference's delta VALUES for every (row, parent) pair it shares."""
    g = ref_golden.case(name, normalized)
    e = torch.from_numpy(g["edge_index"])
    c = cbm_matrix(e, torch.ones(e.shape[1]), alpha=g["alpha"], normalized=normalized)
    assert c.build_info["n_delta"] == g["col"].shape[0]
    c.check_format(e)
    if normalized:
        np.testing.assert_array_equal(c.col_multiplier.numpy(), g["col_multiplier"])
    n = c.num_rows
    ref_parent = np.empty(n, dtype=np.int64)
    for u in range(n + 1):
        ref_parent[g["mst_col"][g["mst_row"][u]:g["mst_row"][u + 1]]] = u
    same = np.nonzero(ref_parent == c._parent)[0]
    assert same.size > 0
    for v in same.tolist():
        np.testing.assert_array_equal(c._dcol[c._crow[v]:c._crow[v + 1]], g["col"][g["crow"][v]:g["crow"][v + 1]])
        np.testing.assert_array_equal(c._dval[c._crow[v]:c._crow[v + 1]], g["val"][g["crow"][v]:g["crow"][v + 1]])


@pytest.mark.parametrize("name", NAMES)
def test_reference_structure_passes_the_schedule_checks(ref_golden, name):
    """The arrays exactly as the reference emitted them are accepted by the plan construction."""
    import ctypes
    from cbm4gnn_b200 import _lib
    from cbm4gnn_b200.cbm import _ptr
    g = ref_golden.case(name, True)
    n = g["x"].shape[0]
    out = [ctypes.c_int32() for _ in range(4)]
    _lib.check(_lib.lib().cbm_b200_schedule_info(n, _ptr(g["mst_row"]), _ptr(g["mst_col"]), _ptr(g["crow"]), _ptr(g["col"]),
                                                _ptr(g["val"]), _ptr(g["col_multiplier"]), None, 0, 0, n,
                                                *[ctypes.byref(o) for o in out]))
    assert out[3].value == n


# ---------------------------------------------------------------------------------------------
# live against the compiled reference (oracle/_ref)
# ---------------------------------------------------------------------------------------------
needs_ref = pytest.mark.skipif(not reference.ref_available(), reason="oracle/_ref has not been built")


def _csr_args(c):
    crow = torch.from_numpy(c._crow)
    return crow[:-1].contiguous(), crow[1:].contiguous(), torch.from_numpy(c._dcol), torch.from_numpy(c._dval)


@needs_ref
@pytest.mark.parametrize("normalized", [False, True])
def test_restatement_equals_compiled_reference_on_config1(normalized):
    ref = reference.ref_module()
    ei = graphs.make_graph("c1")
    if normalized:
        from helpers import with_self_loops
        ei = with_self_loops(ei)
    e = torch.from_numpy(ei)
    c = cbm_matrix(e.to(torch.int32), torch.ones(e.shape[1]), alpha=0 if not normalized else 2, normalized=normalized)
    x = torch.from_numpy(graphs.make_features("c1", c.num_rows, f=96))
    rb, re_, col, val = _csr_args(c)
    for prefix, parallel in (("seq", False), ("omp", True)):
        y = torch.zeros_like(x)
        d = torch.zeros_like(x)
        getattr(ref, f"{prefix}_s_spmm_csr_int32")(rb, re_, col, val, x, d)
        if normalized:
            getattr(ref, f"{prefix}_s_fused_spmm_update_csr_int32")(rb, re_, col, val, x, c.mst_row, c.mst_col, c.col_multiplier, y)
            upd = orc.fused_update(c.mst_row.numpy(), c.mst_col.numpy(), c.col_multiplier.numpy(), d.numpy().copy(), parallel)
            full = orc.fused_spmm_update(c.mst_row.numpy(), c.mst_col.numpy(), c._crow, c._dcol, c._dval,
                                         c.col_multiplier.numpy(), x.numpy(), parallel)
        else:
            getattr(ref, f"{prefix}_s_spmm_update_csr_int32")(rb, re_, col, val, x, c.mst_row, c.mst_col, y)
            upd = orc.update(c.mst_row.numpy(), c.mst_col.numpy(), d.numpy().copy(), parallel)
            full = orc.spmm_update(c.mst_row.numpy(), c.mst_col.numpy(), c._crow, c._dcol, c._dval, x.numpy(), parallel)
        # same delta product in, same update out: bit for bit
        np.testing.assert_array_equal(upd, y.numpy())
        # own summation order in the delta product: the reference's tolerance
        np.testing.assert_allclose(full, y.numpy(), **TOL)


@needs_ref
def test_compiled_reference_builder_agrees_on_config1_weight():
    ref = reference.ref_module()
    ei = graphs.make_graph("c1", scale=0.5)
    order = np.lexsort((ei[1], ei[0]))
    e = torch.from_numpy(np.ascontiguousarray(ei[:, order])).to(torch.int32)
    n = int(e.max()) + 1
    for alpha in (0, 4):
        out = ref.from_coo_int32_t_v1_(e[0].contiguous(), e[1].contiguous(), torch.ones(e.shape[1]), n, n, alpha)
        c = cbm_matrix(e, torch.ones(e.shape[1]), alpha=alpha)
        assert out[4].numel() == c.build_info["n_delta"]
