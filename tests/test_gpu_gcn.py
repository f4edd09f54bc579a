"""GCN layers and the differentiable product against torch sparse autograd (fp32, 1e-4)."""
import numpy as np
import pytest
import torch

from cbm4gnn_b200 import graphs
from cbm4gnn_b200.cbm import cbm_matrix
from cbm4gnn_b200.gcn import (CBMCudaGCN, CBMParallelMKLCSRSparseMatrixGCN, GCNModel)
from cbm4gnn_b200.message_passing import CBMParallelMKLCSRSparseMatrixMessagePassing
from cbm4gnn_b200.utility import add_self_loops, normalize_edge_index

pytestmark = pytest.mark.gpu
TOL = dict(atol=1e-4, rtol=1e-4)


def _er(n, p, f, seed):
    ei = torch.from_numpy(graphs.erdos_renyi(n, p, seed))
    x = torch.randint(0, 10, (int(ei.max()) + 1, f), generator=torch.Generator().manual_seed(seed)).float()
    return ei, x


def test_message_passing_matches_scatter_add():
    """The comparison of tests/test_message_passing.py:53-90: unnormalized, default alpha = 2."""
    ei, x = _er(25, 0.75, 10, 3)
    want = torch.zeros_like(x).index_add_(0, ei[1], x[ei[0]])
    mp = CBMParallelMKLCSRSparseMatrixMessagePassing()
    got = mp.forward(ei.cuda(), x=x.cuda())
    torch.testing.assert_close(got.cpu(), want, **TOL)
    with pytest.raises(ValueError):
        mp.forward(ei.cuda())


def test_two_node_cycle_is_an_involution():
    ei = torch.tensor([[0, 1], [1, 0]])
    x = torch.rand((2, 10))
    mp = CBMParallelMKLCSRSparseMatrixMessagePassing()
    y = mp.forward(ei, x=x.cuda())
    y = mp.forward(ei, x=y)
    torch.testing.assert_close(y.cpu(), x, **TOL)


def test_gcn_layer_forward_and_weight_grad():
    """tests/test_message_passing.py:123-197 checks forward agreement of every GCN layer with the
    scatter-add layer and leaves the CBM backward commented out; here forward and the weight /
    input gradients are checked against torch sparse autograd."""
    ei, x = _er(25, 0.75, 10, 4)
    ei = add_self_loops(ei)
    n = x.size(0)
    layer = CBMParallelMKLCSRSparseMatrixGCN(10, 1).cuda()
    w = layer.lin.weight.detach().cpu().clone().requires_grad_(True)
    a = torch.sparse_coo_tensor(torch.stack([ei[1], ei[0]]), normalize_edge_index(ei), (n, n))
    xr = x.clone().requires_grad_(True)
    want = a @ (xr @ w.t())
    want.sum().backward()
    xg = x.cuda().requires_grad_(True)
    got = layer(xg, ei.cuda())
    got.sum().backward()
    torch.testing.assert_close(got.detach().cpu(), want.detach(), **TOL)
    torch.testing.assert_close(layer.lin.weight.grad.cpu(), w.grad, **TOL)
    torch.testing.assert_close(xg.grad.cpu(), xr.grad, **TOL)


def test_directed_graph_gradient_uses_the_transposed_structure():
    rng = np.random.default_rng(2)
    n = 60
    mask = rng.random((n, n)) < 0.15
    np.fill_diagonal(mask, True)
    ei = torch.from_numpy(np.stack(np.nonzero(mask)))
    c = cbm_matrix(ei.to(torch.int32), torch.ones(ei.shape[1]), alpha=1, normalized=True)
    assert not c.is_symmetric()
    s = c.col_multiplier
    a = torch.sparse_coo_tensor(ei, s[ei[0]] * s[ei[1]], (n, n))
    x = torch.randn((n, 12))
    xr = x.clone().requires_grad_(True)
    g = torch.randn((n, 12))
    (a @ xr).backward(g)
    xg = x.cuda().requires_grad_(True)
    y = c.matmul(xg)
    y.backward(g.cuda())
    torch.testing.assert_close(y.detach().cpu(), (a @ x), **TOL)
    torch.testing.assert_close(xg.grad.cpu(), xr.grad, **TOL)


def test_two_layer_gcn_config3_scaled():
    """Scaled-down stand-in for the 2-layer GCN configuration: SBM graph, widths 128 -> 256 -> 64,
    ReLU between layers, loss = sum of outputs; forward and all gradients against torch sparse."""
    ei_np = graphs.make_graph("c3", scale=0.02)
    ei = add_self_loops(torch.from_numpy(ei_np))
    n = int(ei.max()) + 1
    x = torch.from_numpy(graphs.make_features("c3", n, f=128))
    structure = cbm_matrix(torch.stack([ei[1], ei[0]]).to(torch.int32), torch.ones(ei.shape[1]), alpha=2,
                           normalized=True)
    torch.manual_seed(0)
    model = GCNModel((128, 256, 64), structure=structure).cuda()
    w1 = model.layers[0].lin.weight.detach().cpu().clone().requires_grad_(True)
    w2 = model.layers[1].lin.weight.detach().cpu().clone().requires_grad_(True)
    a = torch.sparse_coo_tensor(torch.stack([ei[1], ei[0]]), normalize_edge_index(ei), (n, n)).coalesce()
    xr = x.clone().requires_grad_(True)
    want = a @ ((a @ (xr @ w1.t())).relu() @ w2.t())
    want.sum().backward()
    xg = x.cuda().requires_grad_(True)
    got = model(xg, ei.cuda())
    got.sum().backward()
    torch.testing.assert_close(got.detach().cpu(), want.detach(), atol=2e-4, rtol=1e-4)
    torch.testing.assert_close(model.layers[0].lin.weight.grad.cpu(), w1.grad, atol=2e-3, rtol=1e-4)
    torch.testing.assert_close(model.layers[1].lin.weight.grad.cpu(), w2.grad, atol=2e-3, rtol=1e-4)
    torch.testing.assert_close(xg.grad.cpu(), xr.grad, atol=2e-4, rtol=1e-4)
    # one structure serves every layer, as benchmark_gcn_cpu.py:62-66 arranges
    assert model.layers[0].cached_a_t is model.layers[1].cached_a_t
