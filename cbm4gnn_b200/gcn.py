"""GCN layers on the CBM product: ``forward(x, edge_index) = propagate(lin(x))``.

Mirrors gnns/graph_convolutional_network/cbm_gcn.py:10-75: a bias-free linear map with
Glorot-uniform weights (the reference uses torch_geometric's ``Linear(..., bias=False,
weight_initializer='glorot')``, restated here on ``torch.nn.Linear`` because torch_geometric is not
available offline) followed by the normalized CBM propagation.  ``GCNModel`` restates the stacked
benchmark model of benchmark/parallel/benchmark_gcn_cpu.py:70-89 (ReLU between layers, one CBM
structure shared by every layer).

The dense map and its gradients run on the tensor cores through the library's fp32-accurate GEMMs
(cbm4gnn_b200/dense.py), so that results stay within the 1e-4 tolerance the reference's tests use.
"""
from __future__ import annotations

import torch
from torch import nn

from .dense import linear, linear_relu, relu_linear_linear
from .message_passing import CBMCudaMessagePassing


def _fp32_linear(lin: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    return linear(x, lin.weight)


class CBMCudaGCN(CBMCudaMessagePassing):
    """``order``: "lin_first" is the reference's ``propagate(lin(x))`` (cbm_gcn.py:21-24);
    "propagate_first" computes ``lin(propagate(x))``, the same matrix product ``A (X W) = (A X) W``
    with the sparse product running at the input width; "auto" (default) propagates at the
    narrower of the two widths."""

    def __init__(self, in_channels: int, out_channels: int, alpha: int = 2, order: str = "auto"):
        super().__init__(normalize=True, alpha=alpha)
        if order not in ("auto", "lin_first", "propagate_first"):
            raise ValueError("order must be 'auto', 'lin_first' or 'propagate_first'")
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.order = order
        self.lin = nn.Linear(in_channels, out_channels, bias=False)
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.xavier_uniform_(self.lin.weight)  # Glorot-uniform

    def propagate_first(self) -> bool:
        return self.order == "propagate_first" or (self.order == "auto" and self.in_channels < self.out_channels)

    def product_width(self) -> int:
        return self.in_channels if self.propagate_first() else self.out_channels

    def propagate_only(self, x, edge_index):
        """The layer's sparse half alone: ``A_hat @ x``."""
        return CBMCudaMessagePassing.forward(self, edge_index, x=x)

    def forward(self, x, edge_index, relu: bool = False):
        """``relu``: apply the ReLU that follows this layer in a stack; when the dense map comes
        last in the layer it runs in the map's epilogue."""
        if self.propagate_first():
            p = super().forward(edge_index, x=x)
            return linear_relu(p, self.lin.weight) if relu else _fp32_linear(self.lin, p)
        x = _fp32_linear(self.lin, x)
        y = super().forward(edge_index, x=x)
        return y.relu() if relu else y


# Reference class names (cbm_gcn.py:10, 27, 44, 61).
class CBMSequentialMKLCSRSparseMatrixGCN(CBMCudaGCN):
    pass


class CBMParallelMKLCSRSparseMatrixGCN(CBMCudaGCN):
    pass


class CBMSequentialTorchCSRSparseMatrixGCN(CBMCudaGCN):
    two_step = True


class CBMParallelTorchCSRSparseMatrixGCN(CBMCudaGCN):
    two_step = True


class GCNModel(nn.Module):
    """``len(widths) - 1`` GCN layers with ReLU between them, sharing one CBM structure."""

    def __init__(self, widths, structure=None, alpha: int = 2):
        super().__init__()
        if len(widths) < 3:
            raise ValueError("Number of layers must be at least 2")
        self.layers = nn.ModuleList(CBMCudaGCN(a, b, alpha=alpha) for a, b in zip(widths[:-1], widths[1:]))
        if structure is not None:
            self.share(structure)

    def product_widths(self):
        """Operand width of each layer's sparse product, in layer order."""
        return [layer.product_width() for layer in self.layers]

    def share(self, structure):
        for layer in self.layers:
            layer.cached_a_t = structure

    def forward(self, x, edge_index):
        """Where a layer that propagates first is followed by one that propagates last, the two dense
        maps and the ReLU between them are adjacent — ``A (relu((A x) W1^T) W2^T)`` — and run as one
        differentiable step (``relu_linear_linear``)."""
        last = len(self.layers) - 1
        i = 0
        while i <= last:
            layer = self.layers[i]
            nxt = self.layers[i + 1] if i < last else None
            if nxt is not None and x.is_cuda and layer.propagate_first() and not nxt.propagate_first():
                p = layer.propagate_only(x, edge_index)
                u = relu_linear_linear(p, layer.lin.weight, nxt.lin.weight)
                x = nxt.propagate_only(u, edge_index)
                if i + 1 < last:
                    x = x.relu()
                i += 2
                continue
            x = layer(x, edge_index, relu=i < last)
            i += 1
        return x
