"""Input-contract checks and graph normalisation helpers.

Restates cbm/utility.py:4-30 (edge_index validators) and gnns/utility.py:4-43 (degree, symmetric
normalisation weights, self loops) of the reference; these define what "normalized" means for the
CBM product and give the weights of the plain-CSR comparison matrix.
"""
from __future__ import annotations

import torch
from torch import Tensor


def check_edge_index_shape(edge_index: Tensor) -> None:
    if edge_index.dim() != 2 or edge_index.shape[0] != 2:
        raise ValueError("Edge index should have shape (2, num_edges)")


def check_edge_index_indices(edge_index: Tensor) -> None:
    if edge_index.numel() and edge_index.min() != 0:
        raise ValueError("Edge index should start from 0")


def check_edge_index_contiguous(edge_index: Tensor) -> None:
    if edge_index.unique().size(0) != edge_index.max() + 1:
        raise ValueError("Edge index is not contiguous")


def check_edge_index_coalesced(edge_index: Tensor) -> None:
    if edge_index.shape[1] != edge_index.unique(dim=1).shape[1]:
        raise ValueError("Edge index is not coalesced")


def check_edge_index(edge_index: Tensor) -> None:
    """All four checks of cbm/utility.py:26-30, in the same order."""
    check_edge_index_shape(edge_index)
    check_edge_index_indices(edge_index)
    check_edge_index_contiguous(edge_index)
    check_edge_index_coalesced(edge_index)


def degree(index: Tensor, num_nodes: int | None = None, dtype=None) -> Tensor:
    """Occurrences of every node id in ``index`` (gnns/utility.py:15-22)."""
    if num_nodes is None:
        num_nodes = int(index.max().item()) + 1
    if dtype is None:
        dtype = index.dtype
    out = torch.zeros((num_nodes,), dtype=dtype, device=index.device)
    return out.scatter_add_(0, index.long(), torch.ones_like(index, dtype=dtype))


def normalize_edge_index(edge_index: Tensor, num_nodes: int | None = None) -> Tensor:
    """Weights ``deg^-1/2[row] * deg^-1/2[col]`` with ``deg`` counted over the second row of
    ``edge_index`` and infinities replaced by 0 (gnns/utility.py:25-33)."""
    if num_nodes is None:
        num_nodes = int(edge_index.max().item()) + 1
    row, col = edge_index[0].long(), edge_index[1].long()
    deg_inv_sqrt = degree(col, num_nodes, torch.float32).pow_(-0.5)
    deg_inv_sqrt[deg_inv_sqrt == float("inf")] = 0
    return deg_inv_sqrt[row] * deg_inv_sqrt[col]


def normalize_torch_adj(a: Tensor) -> Tensor:
    """``D^-1/2 A D^-1/2`` of a sparse adjacency tensor, degrees summed over dim 0
    (gnns/utility.py:4-12); returned as sparse CSR."""
    coo = a.to_sparse_coo().coalesce()
    idx, val = coo.indices(), coo.values()
    deg = torch.zeros(a.shape[1], dtype=val.dtype, device=val.device).scatter_add_(0, idx[1], val)
    dis = deg.pow(-0.5)
    w = dis[idx[0]] * val * dis[idx[1]]
    return torch.sparse_coo_tensor(idx, w, a.shape).coalesce().to_sparse_csr()


def add_self_loops(edge_index: Tensor, num_nodes: int | None = None) -> Tensor:
    """Drop existing self loops, add one per node, coalesce (gnns/utility.py:36-43)."""
    if num_nodes is None:
        num_nodes = int(edge_index.max().item()) + 1
    keep = edge_index[:, edge_index[0] != edge_index[1]]
    loops = torch.arange(num_nodes, dtype=edge_index.dtype, device=edge_index.device).repeat(2, 1)
    both = torch.cat([keep, loops], dim=1).long()
    key = torch.unique(both[0] * num_nodes + both[1])
    return torch.stack([key // num_nodes, key % num_nodes]).to(edge_index.dtype)
