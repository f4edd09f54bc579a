"""Parity at the stated sizes of the benchmark configurations 3, 4 and 5 (synthetic graphs with
those node counts, degree shapes and operand widths), through the C ABI on one GPU.

Configuration 3: forward and every gradient of the 2-layer GCN against torch's sparse autograd on
the full output.  Configurations 4 and 5: the products against a float64 CSR product on a sample of
output rows (the full float64 product of the 35 M- and 57 M-entry matrices would take minutes on
the host), with tolerance atol = rtol = 1e-4 (tests/test_matmul_correctness.py:43).
"""
import numpy as np
import pytest
import torch

from cbm4gnn_b200 import graphs
from cbm4gnn_b200.cbm import cbm_matrix
from cbm4gnn_b200.gcn import GCNModel
from cbm4gnn_b200.utility import add_self_loops, normalize_edge_index

pytestmark = pytest.mark.gpu
TOL = dict(atol=1e-4, rtol=1e-4)


def _row_sample_product(ei, s, rows, x64):
    """float64 rows of D^-1/2 A D^-1/2 @ x for the sampled output rows."""
    import scipy.sparse as sp
    n = x64.shape[0]
    a = sp.csr_matrix((np.ones(ei.shape[1], dtype=np.float64), (ei[0], ei[1])), shape=(n, n))
    sub = a[rows]
    sub = sp.diags(s[rows]) @ sub @ sp.diags(s)
    return sub @ x64


def test_config3_full_size_forward_and_gradients():
    """N = 235 868, widths 128 -> 256 -> 64, ReLU, loss = sum: against torch sparse autograd on the
    GPU (fp32 cuSPARSE products, fp32 GEMMs with TF32 off)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    ei_np = graphs.make_graph("c3")
    ei = add_self_loops(torch.from_numpy(ei_np))
    n = int(ei.max()) + 1
    assert n == 235_868
    x = torch.from_numpy(graphs.make_features("c3", n, f=128)).cuda()
    structure = cbm_matrix(torch.stack([ei[1], ei[0]]).to(torch.int32), torch.ones(ei.shape[1]), alpha=2,
                           normalized=True)
    torch.manual_seed(0)
    model = GCNModel((128, 256, 64), structure=structure).cuda()
    w1 = model.layers[0].lin.weight.detach().clone().double().requires_grad_(True)
    w2 = model.layers[1].lin.weight.detach().clone().double().requires_grad_(True)
    eid = ei.cuda()
    a = torch.sparse_coo_tensor(torch.stack([eid[1], eid[0]]), normalize_edge_index(ei).cuda().double(), (n, n)).coalesce()
    xr = x.double().clone().requires_grad_(True)
    xg = x.clone().requires_grad_(True)
    h1 = model.layers[0](xg, eid)
    got = model.layers[1](h1.relu(), eid)
    got.sum().backward()
    structure.plan().status()
    # The float64 comparison runs through the SAME ReLU mask as the fp32 model: a pre-activation
    # within rounding distance of zero may fall on the other side in float64, which would switch a
    # whole unit on or off and has nothing to do with the accuracy of the products.  The mask may
    # differ from the float64 one only where the float64 pre-activation is that close to zero.
    h1r = torch.sparse.mm(a, xr @ w1.t())
    torch.testing.assert_close(h1.detach().double(), h1r.detach(), **TOL)
    mask = h1.detach() > 0
    assert ((mask != (h1r.detach() > 0)) & (h1r.detach().abs() > 1e-4)).sum().item() == 0
    want = torch.sparse.mm(a, (h1r * mask.double()) @ w2.t())
    want.sum().backward()
    # outputs and input gradient are sums of a few dozen terms: the reference's tolerance;
    # weight gradients sum 235 868 terms each, so their absolute error scales with their size
    torch.testing.assert_close(got.detach().double(), want.detach(), **TOL)
    torch.testing.assert_close(xg.grad.double(), xr.grad, **TOL)
    for mine, ref in ((model.layers[0].lin.weight.grad, w1.grad), (model.layers[1].lin.weight.grad, w2.grad)):
        scale = ref.abs().max().item()
        assert (mine.double() - ref).abs().max().item() <= 1e-4 * scale + 1e-4


@pytest.fixture(scope="module")
def c4_graph():
    ei = add_self_loops(torch.from_numpy(graphs.make_graph("c4"))).numpy()
    n = int(ei.max()) + 1
    x = graphs.make_features("c4", n)
    deg = np.bincount(ei[0], minlength=n).astype(np.float64)
    rows = np.sort(np.random.default_rng(4).choice(n, 2000, replace=False))
    # the highest-degree rows are the ones cut into hundreds of segments: always in the sample
    rows = np.unique(np.concatenate([rows, np.argsort(deg)[-8:]]))
    want = _row_sample_product(ei, deg ** -0.5, rows, x.astype(np.float64))
    return ei, n, x, rows, want


@pytest.mark.parametrize("alpha", [0, 4, 16, 64])
def test_config4_full_size_alpha_sweep(c4_graph, alpha):
    """N = 132 534 copy-model graph (p = 0.95, 20 random links), F = 128, X uniform[-1,1), normalized."""
    ei, n, x, rows, want = c4_graph
    assert n == 132_534
    e = torch.from_numpy(ei).to(torch.int32)
    c = cbm_matrix(e, torch.ones(e.shape[1]), alpha=alpha, normalized=True)
    assert c.build_info["n_delta"] < ei.shape[1]          # the configuration compresses
    xd = torch.from_numpy(x).cuda()
    y = torch.full((n, 128), float("nan"), device="cuda")
    c.omp_mkl_csr_fused_spmm_update(xd, y)
    c.plan().status()
    assert not torch.isnan(y).any()
    np.testing.assert_allclose(y[torch.from_numpy(rows).cuda()].cpu().numpy(), want, **TOL)
    # two-step form (delta product, then the update-only kernel) gives the same rows
    d = torch.empty_like(y)
    c.omp_mkl_csr_spmm(xd, d)
    c.omp_mkl_csr_fused_update(d)
    np.testing.assert_allclose(d[torch.from_numpy(rows).cuda()].cpu().numpy(), want, **TOL)


def test_config5_full_size_per_layer_products():
    """N = 2 449 029 block-model graph, alpha = 2: the products of the 3-layer stack at its two
    distinct operand widths, 256 and 47 (the latter not a multiple of 4: scalar path and the padded
    path of the differentiable product)."""
    ei = add_self_loops(torch.from_numpy(graphs.make_graph("c5"))).numpy()
    n = int(ei.max()) + 1
    assert n == 2_449_029
    e = torch.from_numpy(ei).to(torch.int32)
    c = cbm_matrix(e, torch.ones(e.shape[1]), alpha=2, normalized=True)
    deg = np.bincount(ei[0], minlength=n).astype(np.float64)
    rows = np.sort(np.random.default_rng(5).choice(n, 1500, replace=False))
    rd = torch.from_numpy(rows).cuda()
    for f in (256, 47):
        x = graphs.make_features("c5", n, f=f)
        want = _row_sample_product(ei, deg ** -0.5, rows, x.astype(np.float64))
        xd = torch.from_numpy(x).cuda()
        y = torch.full((n, f), float("nan"), device="cuda")
        c.omp_mkl_csr_fused_spmm_update(xd, y)
        c.plan().status()
        assert not torch.isnan(y).any()
        np.testing.assert_allclose(y[rd].cpu().numpy(), want, **TOL)
        np.testing.assert_allclose(c.matmul(xd)[rd].cpu().numpy(), want, **TOL)
        del xd, y
