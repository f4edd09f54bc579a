"""The dense half of a GCN layer on B200's tensor cores.

A layer of the reference is ``lin`` followed by ``propagate``
(gnns/graph_convolutional_network/cbm_gcn.py:21-24); ``lin`` is a bias-free fp32 map
``[N, in] x [in, out]``.  ``linear(x, weight)`` runs it, and ``autograd`` its two gradients, through
the library's fp32-accurate tensor-core GEMMs (``cbm_b200_dense_forward`` / ``_grad_input`` /
``_grad_weight``: operands split into three bf16 terms, fp32 accumulation), which keep the 1e-4
tolerance of the reference's tests that a single TF32 or BF16 pass would not.  CPU tensors go
through ``torch.nn.functional.linear``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _pad4(v: int) -> int:
    return -(-v // 4) * 4


def _aligned(t: torch.Tensor) -> torch.Tensor:
    """Row-major, 16-byte aligned rows (row stride a multiple of 4 floats): as is, or a copy."""
    if t.stride(1) == 1 and t.stride(0) % 4 == 0 and t.data_ptr() % 16 == 0 and t.stride(0) >= t.size(1):
        return t
    out = torch.empty((t.size(0), _pad4(t.size(1))), dtype=t.dtype, device=t.device)
    out[:, :t.size(1)].copy_(t)
    if out.size(1) != t.size(1):
        out[:, t.size(1):].zero_()
    return out[:, :t.size(1)]


def _widen(t: torch.Tensor, cols: int) -> torch.Tensor:
    """``t`` with zero columns appended up to ``cols`` (a copy only when needed)."""
    t = _aligned(t)
    if t.size(1) == cols:
        return t
    out = torch.zeros((t.size(0), cols), dtype=t.dtype, device=t.device)
    out[:, :t.size(1)].copy_(t)
    return out


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def dense_forward(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, relu: bool = False) -> torch.Tensor:
    """``x @ w.T`` (``relu``: followed by ``max(., 0)`` in the GEMM's epilogue) for CUDA fp32 ``x``
    [N, in] and ``w`` [out, in]; ``out`` (optional) is an [N, out] view with 16-byte aligned rows
    that receives the result."""
    n, n_in, n_out = x.size(0), x.size(1), w.size(0)
    ip, op = _pad4(n_in), _pad4(n_out)
    xa, wa = _widen(x, ip), _widen(w, ip)
    if op != n_out:
        wp = torch.zeros((op, ip), dtype=w.dtype, device=w.device)
        wp[:n_out].copy_(wa)
        wa = wp
    direct = out is not None and op == n_out and out.stride(1) == 1 and out.stride(0) % 4 == 0 and out.data_ptr() % 16 == 0
    y = out if direct else torch.empty((n, op), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        fn = _lib.lib().cbm_b200_dense_forward_relu if relu else _lib.lib().cbm_b200_dense_forward
        _lib.check(fn(xa.data_ptr(), xa.stride(0), wa.data_ptr(), wa.stride(0), y.data_ptr(), y.stride(0), n, ip, op, _stream(x)))
    if direct:
        return out
    y = y[:, :n_out]
    if out is not None:
        out.copy_(y)
        return out
    return y


def dense_grad_input(gy: torch.Tensor, w: torch.Tensor, relu_output: torch.Tensor | None = None) -> torch.Tensor:
    """``gy @ w`` for ``gy`` [N, out], ``w`` [out, in].  With ``relu_output`` [N, in] (the output of
    the ReLU this gradient flows back through) the result is zeroed where that output is zero, in
    the GEMM's epilogue."""
    n, n_out, n_in = gy.size(0), gy.size(1), w.size(1)
    ip, op = _pad4(n_in), _pad4(n_out)
    ga = _widen(gy, op)
    wa = _widen(w, ip)
    if op != n_out:
        wp = torch.zeros((op, ip), dtype=w.dtype, device=w.device)
        wp[:n_out].copy_(wa)
        wa = wp
    gx = torch.empty((n, ip), dtype=gy.dtype, device=gy.device)
    with torch.cuda.device(gy.device):
        if relu_output is None:
            _lib.check(_lib.lib().cbm_b200_dense_grad_input(ga.data_ptr(), ga.stride(0), wa.data_ptr(), wa.stride(0),
                                                            gx.data_ptr(), gx.stride(0), n, ip, op, _stream(gy)))
        else:
            ha = _widen(relu_output, ip)
            _lib.check(_lib.lib().cbm_b200_dense_grad_input_relu(ga.data_ptr(), ga.stride(0), wa.data_ptr(), wa.stride(0),
                                                                 ha.data_ptr(), ha.stride(0), gx.data_ptr(), gx.stride(0),
                                                                 n, ip, op, _stream(gy)))
    return gx[:, :n_in]


_workspaces: dict = {}


def dense_grad_weight(gy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``gy.T @ x`` for ``gy`` [N, out], ``x`` [N, in]: the weight gradient [out, in].  The partial
    results of the row chunks go through one workspace per device, so calls on one device must not
    overlap (autograd issues them on one stream)."""
    n, n_out, n_in = gy.size(0), gy.size(1), x.size(1)
    ip, op = _pad4(n_in), _pad4(n_out)
    ga, xa = _widen(gy, op), _widen(x, ip)
    L = _lib.lib()
    need = int(L.cbm_b200_dense_grad_weight_workspace(n, ip, op))
    ws = _workspaces.get(gy.device)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=gy.device)
        _workspaces[gy.device] = ws
    gw = torch.empty((op, ip), dtype=gy.dtype, device=gy.device)
    with torch.cuda.device(gy.device):
        _lib.check(L.cbm_b200_dense_grad_weight(ga.data_ptr(), ga.stride(0), xa.data_ptr(), xa.stride(0), gw.data_ptr(),
                                                gw.stride(0), n, ip, op, ws.data_ptr(), ws.numel(), _stream(gy)))
    return gw[:n_out, :n_in]


class _DenseMap(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return dense_forward(x, weight)

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        gx = dense_grad_input(gy, weight) if ctx.needs_input_grad[0] else None
        gw = dense_grad_weight(gy, x) if ctx.needs_input_grad[1] else None
        return gx, gw


class _DenseMapRelu(torch.autograd.Function):
    """``relu(x @ w.T)`` with the ReLU in the GEMM's epilogue; the gradient masks with the output."""

    @staticmethod
    def forward(ctx, x, weight):
        h = dense_forward(x, weight, relu=True)
        ctx.save_for_backward(x, weight, h)
        return h

    @staticmethod
    def backward(ctx, gh):
        x, weight, h = ctx.saved_tensors
        gy = torch.ops.aten.threshold_backward(gh, h, 0.0)  # gh where h > 0, else 0: one pass
        gx = dense_grad_input(gy, weight) if ctx.needs_input_grad[0] else None
        gw = dense_grad_weight(gy, x) if ctx.needs_input_grad[1] else None
        return gx, gw


def linear_relu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``relu(x @ weight.T)`` in fp32 accuracy, differentiable in both arguments."""
    if not x.is_cuda:
        return torch.nn.functional.linear(x, weight).relu()
    if x.dtype != torch.float32 or weight.dtype != torch.float32:
        raise RuntimeError("dense map: fp32 operands expected")
    return _DenseMapRelu.apply(x, weight)


class _ReluMapThenMap(torch.autograd.Function):
    """``relu(p @ w1.T) @ w2.T``: the dense map that ends one layer, the ReLU between two layers and
    the dense map that opens the next one.  Forward: the ReLU in the first map's epilogue.
    Backward: the ReLU's mask in the epilogue of the second map's input gradient, so the hidden
    activations are never passed over by an elementwise kernel in either direction."""

    @staticmethod
    def forward(ctx, p, w1, w2):
        h = dense_forward(p, w1, relu=True)
        ctx.save_for_backward(p, w1, w2, h)
        return dense_forward(h, w2)

    @staticmethod
    def backward(ctx, gu):
        p, w1, w2, h = ctx.saved_tensors
        gw2 = dense_grad_weight(gu, h) if ctx.needs_input_grad[2] else None
        gp = gw1 = None
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            gz = dense_grad_input(gu, w2, relu_output=h)  # gradient at the first map's output, before its ReLU
            gp = dense_grad_input(gz, w1) if ctx.needs_input_grad[0] else None
            gw1 = dense_grad_weight(gz, p) if ctx.needs_input_grad[1] else None
        return gp, gw1, gw2


def relu_linear_linear(p: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """``relu(p @ w1.T) @ w2.T`` in fp32 accuracy, differentiable in all three arguments."""
    if not p.is_cuda:
        return torch.nn.functional.linear(torch.nn.functional.linear(p, w1).relu(), w2)
    if p.dtype != torch.float32 or w1.dtype != torch.float32 or w2.dtype != torch.float32:
        raise RuntimeError("dense map: fp32 operands expected")
    return _ReluMapThenMap.apply(p, w1, w2)


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T`` in fp32 accuracy, differentiable in both arguments."""
    if not x.is_cuda:
        return torch.nn.functional.linear(x, weight)
    if x.dtype != torch.float32 or weight.dtype != torch.float32:
        raise RuntimeError("dense map: fp32 operands expected")
    return _DenseMap.apply(x, weight)
