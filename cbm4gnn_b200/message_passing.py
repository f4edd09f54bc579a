"""CBM message-passing layers: ``out = A^T x`` with the adjacency held as a ``cbm_matrix``.

Mirrors gnns/message_passing/cbm_message_passing.py:7-107 of the reference: the layer transposes
``edge_index`` to ``[dst, src]``, builds the CBM structure once and caches it in ``cached_a_t``
(assignable from outside, as benchmark/parallel/benchmark_gcn_cpu.py:62-66 does to share one
structure between layers), and dispatches to the normalized or plain product.  The four reference
class names are kept; there the ``MKL`` classes call the one-step product and the ``Torch`` classes
the two-step path (``deltas @ x`` then the in-place update, cbm_message_passing.py:80-107), and the
same distinction is kept here on the CUDA kernels (``two_step``).  Unlike the reference, the output is a fresh tensor on
every call (the reference caches and aliases one output buffer, cbm_message_passing.py:26-29), and
the product is differentiable with respect to ``x``.
"""
from __future__ import annotations

import torch
from torch import nn

from .cbm import cbm_matrix


class CBMCudaMessagePassing(nn.Module):
    def __init__(self, flow: str = "source_to_target", node_dim: int = 0, alpha: int = 2,
                 normalize: bool = False, cached: bool = True):
        super().__init__()
        if flow not in ("source_to_target", "target_to_source"):
            raise ValueError(f"Expected 'flow' to be either 'source_to_target' or 'target_to_source' (got '{flow}')")
        self.flow = flow
        self.node_dim = node_dim
        self.normalize = normalize
        self.cached = cached
        self.alpha = alpha
        self.cached_a_t = None

    two_step = False  # True: delta product, then the update-only kernel

    def _structure(self, edge_index: torch.Tensor, dtype, device=None) -> cbm_matrix:
        if self.cached and self.cached_a_t is not None:
            return self.cached_a_t
        edge_index_t = torch.stack([edge_index[1], edge_index[0]], dim=0).to(torch.int32)
        # the builder's candidate search runs on the GPU that holds the features (same structure,
        # several times faster on high-degree graphs)
        build_device = device.index if device is not None and device.type == "cuda" else None
        if build_device is None and device is not None and device.type == "cuda":
            build_device = torch.cuda.current_device()
        a_t = cbm_matrix(edge_index_t, torch.ones(edge_index.size(1), dtype=dtype),
                         normalized=self.normalize, alpha=self.alpha, build_device=build_device)
        if self.cached:
            self.cached_a_t = a_t
        return a_t

    def forward(self, edge_index, size=None, **kwargs):
        if "x" not in kwargs:
            raise ValueError("x must be in kwargs")
        x = kwargs["x"]
        return self._structure(edge_index, x.dtype, x.device).matmul(x, two_step=self.two_step)


# Reference class names (cbm_message_passing.py:7, 39, 63, 90).
class CBMSequentialMKLCSRSparseMatrixMessagePassing(CBMCudaMessagePassing):
    pass


class CBMParallelMKLCSRSparseMatrixMessagePassing(CBMCudaMessagePassing):
    pass


class CBMSequentialTorchCSRSparseMatrixMessagePassing(CBMCudaMessagePassing):
    two_step = True


class CBMParallelTorchCSRSparseMatrixMessagePassing(CBMCudaMessagePassing):
    two_step = True
