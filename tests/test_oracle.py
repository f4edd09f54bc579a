"""The CPU restatement against the fixtures and against dense A @ X (no GPU needed).

Tolerance: atol = rtol = 1e-4 in fp32, the figure of the reference's own tests
(tests/test_matmul_correctness.py:43).
"""
import numpy as np
import pytest

from cbm4gnn_b200 import graphs
from oracle import cbm_oracle as orc
from conftest import golden_case
from helpers import dense_product, with_self_loops

TOL = dict(atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("k", range(5))
@pytest.mark.parametrize("alpha", [0, 2, 3])
def test_oracle_matches_golden_unnormalized(golden, k, alpha):
    ei, x, y, _ = golden_case(golden, k)
    s = orc.build_structure(ei, alpha)
    rows = orc.reconstruct_rows(s["n"], s["mst_row"], s["mst_col"], s["crow"], s["col"], s["val"])
    want = [set(ei[1][ei[0] == r].tolist()) for r in range(s["n"])]
    assert rows == want
    for parallel in (False, True):
        got = orc.spmm_update(s["mst_row"], s["mst_col"], s["crow"], s["col"], s["val"], x, parallel)
        # integer-valued features: the product is exact in fp32
        np.testing.assert_array_equal(got, y)


@pytest.mark.parametrize("k", range(5))
def test_oracle_matches_golden_normalized(golden, k):
    ei, x, _, y_norm = golden_case(golden, k)
    ei = with_self_loops(ei)
    n = x.shape[0]
    mult = orc.row_multiplier(ei, n)
    s = orc.build_structure(ei, 2, col_mul=mult)
    for parallel in (False, True):
        got = orc.fused_spmm_update(s["mst_row"], s["mst_col"], s["crow"], s["col"], s["val"], mult, x, parallel)
        np.testing.assert_allclose(got, y_norm, **TOL)


def test_oracle_two_step_equals_one_step(golden):
    ei, x, y, _ = golden_case(golden, 2)
    s = orc.build_structure(ei, 1)
    d = orc.csr_spmm(s["crow"], s["col"], s["val"], x)
    np.testing.assert_array_equal(orc.update(s["mst_row"], s["mst_col"], d.copy()), y)
    np.testing.assert_array_equal(orc.update(s["mst_row"], s["mst_col"], d.copy(), parallel=True), y)


def test_oracle_copy_model_graph():
    ei = graphs.make_graph("c1", scale=0.1)
    n = int(ei.max()) + 1
    x = graphs.make_features("c1", n, f=33)
    s = orc.build_structure(ei, 0)
    assert s["weight"] <= ei.shape[1]
    got = orc.spmm_update(s["mst_row"], s["mst_col"], s["crow"], s["col"], s["val"], x, True)
    np.testing.assert_allclose(got, dense_product(ei, x, False), **TOL)


def test_oracle_arborescence_is_optimal_small():
    nx = pytest.importorskip("networkx")
    for seed in range(4):
        ei = graphs.erdos_renyi(18, 0.45, 100 + seed)
        n = int(ei.max()) + 1
        edges = orc.candidate_edges(ei, n, 1)
        sol = orc.min_arborescence(n + 1, n, edges)
        g = nx.DiGraph()
        for u, v, w in edges:
            if not g.has_edge(u, v) or g[u][v]["weight"] > w:
                g.add_edge(u, v, weight=w)
        ref = nx.minimum_spanning_arborescence(g)
        assert sum(w for _, w in sol.values()) == sum(d["weight"] for _, _, d in ref.edges(data=True))
