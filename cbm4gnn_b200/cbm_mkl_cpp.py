"""Drop-in for the reference's native module ``cbm.cbm_mkl_cpp`` on top of ``libcbm_b200.so``.

The 13 functions bound at cbm/cbm_extensions.cpp:1757-1771 are offered under their own names with
their own argument lists, so the reference's unmodified Python layer (cbm/cbm.py,
gnns/message_passing/cbm_message_passing.py) runs on the CUDA engine once this module is put in its
place::

    import sys, cbm4gnn_b200.cbm_mkl_cpp as shim
    sys.modules["cbm.cbm_mkl_cpp"] = shim      # before `from cbm.cbm import cbm_matrix`

The two builders run on the host (``cbm_b200_build``) and return the reference's five tensors in
its layout.  The eleven compute functions take the CSR/tree arrays on every call, as the reference
passes them; the device schedule derived from them is cached, keyed by the identity and content
fingerprint of the arrays, so only the first call of a structure pays for it.  ``seq_`` and
``omp_`` names run the same kernels.  Dense operands may be CPU tensors (staged through the GPU,
results copied back into ``dst``) or CUDA tensors; index tensors are read on the host.

dtype contract and error wording follow the TORCH_CHECKs of cbm/cbm_extensions.cpp:659-666.
"""
from __future__ import annotations

import ctypes
import zlib

import numpy as np
import torch

from . import _lib
from .cbm import _Plan, _dense_args, _ptr

__all__ = [
    "from_coo_int32_t_v1_", "from_coo_int32_t_v2_",
    "seq_s_spmm_update_csr_int32", "seq_s_update_csr_int32", "seq_s_spmm_csr_int32",
    "omp_s_spmm_update_csr_int32", "omp_s_update_avx_int32", "omp_s_update_csr_int32", "omp_s_spmm_csr_int32",
    "omp_s_fused_spmm_update_csr_int32", "omp_s_fused_update_csr_int32",
    "seq_s_fused_spmm_update_csr_int32", "seq_s_fused_update_csr_int32",
]


def _need(t: torch.Tensor, dtype, name: str, what: str) -> None:
    if t.dtype != dtype:
        raise RuntimeError(f"{name} tensor (NOT torch::{what})")


def _host_i32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().numpy(), dtype=np.int32)


def _host_f32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().numpy(), dtype=np.float32)


# ------------------------------------------------------------------------------------- builders
def _build(src_row, src_col, col_mul, n_rows, n_cols, alpha):
    _need(src_row, torch.int32, "src_row", "kInt32")
    _need(src_col, torch.int32, "src_col", "kInt32")
    if int(n_rows) != int(n_cols):
        raise RuntimeError("the CBM builder takes a square matrix")
    n = int(n_rows)
    row, col = _host_i32(src_row), _host_i32(src_col)
    mul = None if col_mul is None else _host_f32(col_mul)
    L = _lib.lib()
    h = ctypes.c_void_p(0)
    _lib.check(L.cbm_b200_build(_ptr(row), _ptr(col), row.shape[0], n, int(alpha), _ptr(mul), 0, ctypes.byref(h)))
    try:
        n_delta = ctypes.c_int64()
        _lib.check(L.cbm_b200_built_info(h, ctypes.byref(n_delta), None, None, None, None))
        nd = n_delta.value
        mst_row, mst_col = np.empty(n + 2, dtype=np.int32), np.empty(n, dtype=np.int32)
        crow, ccol, cval = np.empty(n + 1, dtype=np.int32), np.empty(nd, dtype=np.int32), np.empty(nd, dtype=np.float32)
        _lib.check(L.cbm_b200_built_export_csr(h, _ptr(mst_row), _ptr(mst_col), _ptr(crow), _ptr(ccol), _ptr(cval), None))
        d_row, d_col, d_val = np.empty(nd, dtype=np.int32), np.empty(nd, dtype=np.int32), np.empty(nd, dtype=np.float32)
        _lib.check(L.cbm_b200_built_export_coo(h, _ptr(d_row), _ptr(d_col), _ptr(d_val)))
    finally:
        L.cbm_b200_built_free(h)
    return [torch.from_numpy(a) for a in (mst_row, mst_col, d_row, d_col, d_val)]


def from_coo_int32_t_v1_(src_row, src_col, src_val, src_n_rows, src_n_cols, alpha):
    """cbm_init_v1_ (cbm/cbm_extensions.cpp:8-326): [edges_row, edges_col, delta_row, delta_col,
    delta_val] with deltas of +-1 as COO triples in breadth-first order of the tree."""
    return _build(src_row, src_col, None, src_n_rows, src_n_cols, alpha)


def from_coo_int32_t_v2_(src_row, src_col, src_val, col_mul, src_n_rows, src_n_cols, alpha):
    """cbm_init_v2_ (cbm/cbm_extensions.cpp:328-644): the same with delta values +-col_mul[col]."""
    _need(col_mul, torch.float32, "col_mul", "kFloat32")
    return _build(src_row, src_col, col_mul, src_n_rows, src_n_cols, alpha)


# --------------------------------------------------------------------------------- plan caching
_plans: dict = {}
_MAX_PLANS = 16


def _fingerprint(*arrays) -> tuple:
    out = []
    for a in arrays:
        if a is None:
            out.append(None)
        else:
            out.append((a.shape[0], zlib.crc32(a.view(np.uint8))))
    return tuple(out)


def _plan_for(device_index, edges_src, edges_dst, row_b=None, row_e=None, col=None, val=None, mul=None) -> _Plan:
    """The device schedule for the given arrays.  The reference passes fresh ``.to(torch.int32)``
    copies on every call (cbm/cbm.py:145-153), so tensors cannot be recognised by address alone:
    the key is a CRC of the contents (microseconds per megabyte, against milliseconds for a new
    schedule)."""
    _need(edges_src, torch.int32, "edges_src", "kInt32")
    _need(edges_dst, torch.int32, "edges_dst", "kInt32")
    mr, mc = _host_i32(edges_src), _host_i32(edges_dst)
    n = mc.shape[0]
    if row_b is not None:
        for t, nm in ((row_b, "lhs_row_b"), (row_e, "lhs_row_e"), (col, "lhs_col")):
            _need(t, torch.int32, nm, "kInt32")
        _need(val, torch.float32, "lhs_val", "kFloat32")
        rb, re_, cc, vv = _host_i32(row_b), _host_i32(row_e), _host_i32(col), _host_f32(val)
        m_rows = rb.shape[0]
        if m_rows > n or re_.shape[0] != m_rows:
            raise RuntimeError("lhs_row_b / lhs_row_e must have one entry per matrix row")
        if m_rows > 1 and not np.array_equal(rb[1:], re_[:-1]):
            raise RuntimeError("lhs_row_b / lhs_row_e must describe one contiguous CSR (row_e[i] == row_b[i+1])")
        if m_rows and rb[0] != 0:
            raise RuntimeError("lhs_row_b must start at 0")
        # cbm/cbm.py:121 sizes the delta tensor by the largest index present, so trailing rows
        # without deltas are missing from the CSR it hands over: they are empty rows
        crow = np.full(n + 1, re_[-1] if m_rows else 0, dtype=np.int32)
        crow[:m_rows] = rb
    else:  # update-only calls carry no deltas: an empty delta matrix
        crow, cc, vv = np.zeros(n + 1, dtype=np.int32), np.zeros(0, dtype=np.int32), np.zeros(0, dtype=np.float32)
    m = None if mul is None else _host_f32(mul)
    key = (device_index,) + _fingerprint(mr, mc, crow, cc, vv, m)
    p = _plans.get(key)
    if p is None:
        if len(_plans) >= _MAX_PLANS:
            _plans.pop(next(iter(_plans)))
        p = _Plan(n, mr, mc, crow, cc, vv, m, device_index)
        _plans[key] = p
    return p


def _device_index(dst: torch.Tensor) -> int:
    if not torch.cuda.is_available():
        raise RuntimeError("cbm4gnn_b200 needs a CUDA device: there is no CPU implementation of the products")
    return dst.device.index if dst.is_cuda and dst.device.index is not None else torch.cuda.current_device()


def _run(fn_name, plan: _Plan, rhs, dst, n):
    _need(dst, torch.float32, "dst", "kFloat32")
    if rhs is not None:
        _need(rhs, torch.float32, "rhs", "kFloat32")
        if rhs.size(0) != n or rhs.size(1) != dst.size(1):
            raise RuntimeError("rhs and dst shapes do not fit the matrix")
    if dst.size(0) != n:
        raise RuntimeError("dst must have one row per matrix row")
    dev = torch.device("cuda", plan.device_index)
    on_host = not dst.is_cuda
    y = dst.to(dev) if on_host else dst
    x = None if rhs is None else (rhs.to(dev) if not rhs.is_cuda else rhs)
    f = int(y.size(1))
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    yp, ldy = _dense_args(y)
    fn = getattr(_lib.lib(), fn_name)
    if x is None:
        _lib.check(fn(plan.handle, yp, ldy, f, stream))
    else:
        xp, ldx = _dense_args(x.contiguous())
        _lib.check(fn(plan.handle, xp, ldx, yp, ldy, f, stream))
    if on_host:
        dst.copy_(y)
        plan.status(stream.value or 0)


# ------------------------------------------------------------------------------ compute surface
def seq_s_spmm_update_csr_int32(lhs_row_b, lhs_row_e, lhs_col, lhs_val, rhs, edges_src, edges_dst, dst):
    """dst = A rhs (cbm/cbm_extensions.cpp:650-740)."""
    p = _plan_for(_device_index(dst), edges_src, edges_dst, lhs_row_b, lhs_row_e, lhs_col, lhs_val)
    _run("cbm_b200_spmm_update", p, rhs, dst, p.n)


def seq_s_update_csr_int32(edges_src, edges_dst, dst):
    """In place: every row of dst gets its tree parent's finished row added (cbm/cbm_extensions.cpp:742-786)."""
    p = _plan_for(_device_index(dst), edges_src, edges_dst)
    _run("cbm_b200_update", p, None, dst, p.n)


def seq_s_spmm_csr_int32(lhs_row_b, lhs_row_e, lhs_col, lhs_val, rhs, dst):
    """dst = M rhs for a plain CSR, no tree (cbm/cbm_extensions.cpp:790-843)."""
    for t, nm in ((lhs_row_b, "lhs_row_b"), (lhs_row_e, "lhs_row_e"), (lhs_col, "lhs_col")):
        _need(t, torch.int32, nm, "kInt32")
    _need(lhs_val, torch.float32, "lhs_val", "kFloat32")
    _need(rhs, torch.float32, "rhs", "kFloat32")
    _need(dst, torch.float32, "dst", "kFloat32")
    dev = torch.device("cuda", _device_index(dst))
    on_host = not dst.is_cuda
    y = dst.to(dev) if on_host else dst
    x = (rhs if rhs.is_cuda else rhs.to(dev)).contiguous()
    rb, re_, col, val = (t.to(dev).contiguous() for t in (lhs_row_b, lhs_row_e, lhs_col, lhs_val))
    n, f = int(y.size(0)), int(y.size(1))
    xp, ldx = _dense_args(x)
    yp, ldy = _dense_args(y)
    _lib.check(_lib.lib().cbm_b200_csr_spmm(n, _ptr(rb), _ptr(re_), _ptr(col), _ptr(val), xp, ldx, yp, ldy, f,
                                            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    if on_host:
        dst.copy_(y)


def seq_s_fused_spmm_update_csr_int32(lhs_row_b, lhs_row_e, lhs_col, lhs_val, rhs, edges_src, edges_dst, mul, dst):
    """dst = D^-1/2 A D^-1/2 rhs (cbm/cbm_extensions.cpp:845-996)."""
    _need(mul, torch.float32, "mul", "kFloat32")
    p = _plan_for(_device_index(dst), edges_src, edges_dst, lhs_row_b, lhs_row_e, lhs_col, lhs_val, mul)
    _run("cbm_b200_fused_spmm_update", p, rhs, dst, p.n)


def seq_s_fused_update_csr_int32(edges_src, edges_dst, mul, dst):
    """In place, normalized tree update y_v = (y_v + y_u / s_u) s_v (cbm/cbm_extensions.cpp:998-1105)."""
    _need(mul, torch.float32, "mul", "kFloat32")
    p = _plan_for(_device_index(dst), edges_src, edges_dst, mul=mul)
    _run("cbm_b200_fused_update", p, None, dst, p.n)


# the OpenMP forms (cbm/cbm_extensions.cpp:1108-1755) run the same kernels
omp_s_spmm_update_csr_int32 = seq_s_spmm_update_csr_int32
omp_s_update_csr_int32 = seq_s_update_csr_int32
omp_s_update_avx_int32 = seq_s_update_csr_int32
omp_s_spmm_csr_int32 = seq_s_spmm_csr_int32
omp_s_fused_spmm_update_csr_int32 = seq_s_fused_spmm_update_csr_int32
omp_s_fused_update_csr_int32 = seq_s_fused_update_csr_int32
