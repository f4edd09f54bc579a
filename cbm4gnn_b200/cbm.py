"""``cbm_matrix`` — the compressed-binary-matrix object, with its products running on B200.

Mirrors the public surface of the reference class (cbm/cbm.py:9-275): same constructor, same
attributes (``deltas``, ``mst_row``, ``mst_col``, ``col_multiplier``), same method names.  The
structure is built on the host by ``libcbm_b200.so`` (replacing ``cbm_mkl_cpp.from_coo_int32_t_v1_``
/ ``_v2_``); every product runs as a CUDA kernel through the same library.  There is no CPU
implementation of the products in this package: a CPU tensor is staged through the GPU by the
library's host-buffer entry point, and a missing library or GPU raises.

Differences from the reference that are deliberate:
* int32 copies of the CSR indices are made once at construction, not on every call
  (cbm/cbm.py:145-148 converts per call);
* ``deltas`` always has shape ``(n, n)`` (the reference infers it from the largest index present,
  cbm/cbm.py:121);
* nothing is printed;
* ``seq_*`` and ``omp_*`` methods run the same kernels — on a GPU there is no thread-count knob;
* ``matmul`` and ``transposed`` are additions: the differentiable product used by the CUDA layers
  and the structure its gradient runs on.
"""
from __future__ import annotations

import ctypes
import warnings
from collections import deque

import numpy as np
import torch

from . import _lib

warnings.filterwarnings("ignore", message="Sparse CSR tensor support is in beta state", category=UserWarning)
warnings.filterwarnings("ignore", message="Sparse invariant checks are implicitly disabled", category=UserWarning)


def _ptr(a) -> ctypes.c_void_p:
    if a is None:
        return ctypes.c_void_p(0)
    if isinstance(a, np.ndarray):
        return ctypes.c_void_p(a.ctypes.data)
    return ctypes.c_void_p(a.data_ptr())


def _as_i32(a) -> np.ndarray:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.int32)


def _as_f32(a) -> np.ndarray:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=np.float32)


def aligned_rows(rows: int, width: int, device, dtype=torch.float32) -> torch.Tensor:
    """A zero-initialised ``[rows, width]`` view whose row pitch is a whole number of 128-byte lines:
    the layout in which a dense operand or result of the products is best kept on the GPU (every
    gathered row piece then fills whole lines; 7-18 % faster products than with a pitch of 500
    floats).  Any row-major tensor is accepted; this is the recommended way to allocate one."""
    pitch = -(-width // 32) * 32
    return torch.zeros((rows, pitch), dtype=dtype, device=device)[:, :width]


class _Plan:
    """Owns one ``cbm_b200_plan`` handle (a device-side schedule for one GPU)."""

    def __init__(self, n, mst_row, mst_col, crow, col, val, multiplier, device_index, perm=None,
                 n_labels=0, own_begin=0, own_end=None):
        L = _lib.lib()
        self.handle = ctypes.c_void_p(0)
        self.device_index = device_index
        own_end = (n_labels or n) if own_end is None else own_end
        perm = None if perm is None else np.ascontiguousarray(perm, dtype=np.int32)
        _lib.check(L.cbm_b200_plan_create(n, _ptr(mst_row), _ptr(mst_col), _ptr(crow), _ptr(col),
                                          _ptr(val), _ptr(multiplier), _ptr(perm), n_labels, own_begin,
                                          own_end, device_index, ctypes.byref(self.handle)))
        n_rows, n_delta = ctypes.c_int32(), ctypes.c_int64()
        n_rc, depth, nbytes = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int64()
        _lib.check(L.cbm_b200_plan_info(self.handle, ctypes.byref(n_rows), ctypes.byref(n_delta),
                                        ctypes.byref(n_rc), ctypes.byref(depth), ctypes.byref(nbytes)))
        self.n = n
        self.n_rows, self.n_delta = n_rows.value, n_delta.value
        self.n_root_children, self.depth, self.device_bytes = n_rc.value, depth.value, nbytes.value

    def tune(self, slab_width=0, n_blocks=0, host_chunk=0, form=0):
        _lib.check(_lib.lib().cbm_b200_plan_tune(self.handle, slab_width, n_blocks, host_chunk, form))

    def status(self, stream=0):
        _lib.check(_lib.lib().cbm_b200_plan_status(self.handle, ctypes.c_void_p(stream)))

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().cbm_b200_plan_destroy(self.handle)
                self.handle = ctypes.c_void_p(0)
        except Exception:
            pass


def _check_f32(name: str, t: torch.Tensor) -> None:
    if t.dtype != torch.float32:
        # same wording as the TORCH_CHECKs of cbm/cbm_extensions.cpp:663-664
        raise RuntimeError(f"{name} tensor (NOT torch::kFloat32)")


def _dense_args(t: torch.Tensor):
    if t.dim() != 2 or t.stride(1) != 1 or (t.size(0) > 1 and t.stride(0) < t.size(1)):
        raise RuntimeError("dense operands must be 2-D and row-major with unit column stride")
    return _ptr(t), int(t.stride(0)) if t.size(0) > 1 else int(t.size(1))


class cbm_matrix:
    def __init__(self, edge_index, values, rows=None, cols=None, alpha=0, normalized=False,
                 deltas_format="csr", n_threads=0, build_device=None):
        """``build_device``: CUDA device ordinal on which to run the builder's candidate search
        (the structure comes out identical; on high-degree graphs the search is nearly all of the
        build time); None = host."""
        ei = edge_index.detach().cpu() if isinstance(edge_index, torch.Tensor) else torch.as_tensor(edge_index)
        if ei.dim() != 2 or ei.size(0) != 2:
            raise ValueError("Edge index should have shape (2, num_edges)")
        row = _as_i32(ei[0])
        col = _as_i32(ei[1])
        # square matrix sized by the largest index present (cbm/cbm.py:15)
        n = int(max(row.max(initial=-1), col.max(initial=-1))) + 1
        self.alpha = int(alpha)
        self.normalized = bool(normalized)
        self.num_rows = n
        self.nnz = int(row.shape[0])

        if not normalized:
            self.col_multiplier = None
            mul = None
        else:
            # D^-1/2 from the row degrees of a binary matrix (cbm/cbm.py:34-41); a row without
            # entries gets inf exactly as there.
            deg = torch.from_numpy(np.bincount(row, minlength=n).astype(np.float32))
            self.col_multiplier = deg.pow(-0.5)
            mul = _as_f32(self.col_multiplier)

        self._build(row, col, n, mul, n_threads, build_device)
        self._symmetric = None
        self._row, self._col = row, col
        self._plans: dict[int, _Plan] = {}
        self._transposed: "cbm_matrix | None" = None

        crow64 = torch.from_numpy(self._crow.astype(np.int64))
        col64 = torch.from_numpy(self._dcol.astype(np.int64))
        val = torch.from_numpy(self._dval)
        csr = torch.sparse_csr_tensor(crow64, col64, val, size=(n, n), check_invariants=False)
        if deltas_format == "coo":
            self.deltas = csr.to_sparse_coo()
        else:  # the reference falls back to csr for anything else (cbm/cbm.py:64-66)
            self.deltas = csr

    # ------------------------------------------------------------------ construction
    def _build(self, row, col, n, mul, n_threads, build_device=None):
        L = _lib.lib()
        h = ctypes.c_void_p(0)
        if build_device is None:
            _lib.check(L.cbm_b200_build(_ptr(row), _ptr(col), row.shape[0], n, self.alpha, _ptr(mul),
                                        int(n_threads), ctypes.byref(h)))
        else:
            _lib.check(L.cbm_b200_build_gpu(_ptr(row), _ptr(col), row.shape[0], n, self.alpha, _ptr(mul),
                                            int(n_threads), int(build_device), ctypes.byref(h)))
        try:
            n_delta, n_cand = ctypes.c_int64(), ctypes.c_int64()
            n_rc, depth = ctypes.c_int32(), ctypes.c_int32()
            secs = (ctypes.c_double * 4)()
            _lib.check(L.cbm_b200_built_info(h, ctypes.byref(n_delta), ctypes.byref(n_cand),
                                             ctypes.byref(n_rc), ctypes.byref(depth), secs))
            nd = n_delta.value
            mst_row = np.empty(n + 2, dtype=np.int32)
            mst_col = np.empty(n, dtype=np.int32)
            crow = np.empty(n + 1, dtype=np.int32)
            dcol = np.empty(nd, dtype=np.int32)
            dval = np.empty(nd, dtype=np.float32)
            parent = np.empty(n, dtype=np.int32)
            _lib.check(L.cbm_b200_built_export_csr(h, _ptr(mst_row), _ptr(mst_col), _ptr(crow),
                                                   _ptr(dcol), _ptr(dval), _ptr(parent)))
            on_gpu = L.cbm_b200_built_candidates_on_gpu(h)
        finally:
            L.cbm_b200_built_free(h)
        self.mst_row = torch.from_numpy(mst_row)
        self.mst_col = torch.from_numpy(mst_col)
        self._crow, self._dcol, self._dval, self._parent = crow, dcol, dval, parent
        self.build_info = dict(n_delta=nd, n_candidates=n_cand.value, n_root_children=n_rc.value,
                               depth=depth.value, seconds_candidates=secs[0],
                               seconds_arborescence=secs[1], seconds_deltas=secs[2],
                               seconds_total=secs[3], candidates_on_gpu=bool(on_gpu))

    @classmethod
    def from_arrays(cls, mst_row, mst_col, delta_crow, delta_col, delta_val, col_multiplier=None):
        """Wrap a structure that already exists in the reference's layout (for instance one built
        by the reference itself): the arrays are consumed unmodified."""
        self = cls.__new__(cls)
        self.mst_row = torch.as_tensor(_as_i32(mst_row))
        self.mst_col = torch.as_tensor(_as_i32(mst_col))
        n = self.mst_col.numel()
        self.num_rows = n
        self.alpha = None
        self._crow, self._dcol, self._dval = _as_i32(delta_crow), _as_i32(delta_col), _as_f32(delta_val)
        self.normalized = col_multiplier is not None
        self.col_multiplier = None if col_multiplier is None else torch.as_tensor(_as_f32(col_multiplier))
        parent = np.empty(n, dtype=np.int32)
        mr, mc = self.mst_row.numpy(), self.mst_col.numpy()
        for u in range(n + 1):
            parent[mc[mr[u]:mr[u + 1]]] = u
        self._parent = parent
        self._symmetric, self._row, self._col = False, None, None
        self._plans, self._transposed = {}, None
        self.build_info = dict(n_delta=int(self._crow[-1]))
        self.nnz = None
        self.deltas = torch.sparse_csr_tensor(torch.from_numpy(self._crow.astype(np.int64)),
                                              torch.from_numpy(self._dcol.astype(np.int64)),
                                              torch.from_numpy(self._dval), size=(n, n), check_invariants=False)
        return self

    # ------------------------------------------------------------------ persistence
    def state_dict(self) -> dict:
        """Everything needed to rebuild this object without running the builder: the tree, the
        delta CSR and the multiplier in the reference's layout, plus the build parameters."""
        return dict(format="cbm4gnn_b200/1", num_rows=self.num_rows, alpha=self.alpha, normalized=self.normalized,
                    nnz=self.nnz, mst_row=self.mst_row.clone(), mst_col=self.mst_col.clone(),
                    delta_crow=torch.from_numpy(self._crow.copy()), delta_col=torch.from_numpy(self._dcol.copy()),
                    delta_val=torch.from_numpy(self._dval.copy()),
                    col_multiplier=None if self.col_multiplier is None else self.col_multiplier.clone(),
                    edge_row=None if self._row is None else torch.from_numpy(self._row.copy()),
                    edge_col=None if self._col is None else torch.from_numpy(self._col.copy()),
                    build_info=dict(self.build_info))

    def save(self, path) -> None:
        """Write the built structure to ``path`` (the build is the expensive step: 20-60 s for
        the high-degree configuration against under a millisecond per product)."""
        torch.save(self.state_dict(), path)

    @classmethod
    def load(cls, path) -> "cbm_matrix":
        """Rebuild an object written by ``save``; the arrays are used exactly as stored."""
        st = torch.load(path, map_location="cpu", weights_only=True)  # tensors and plain values only
        if st.get("format") != "cbm4gnn_b200/1":
            raise ValueError(f"{path}: not a saved cbm_matrix")
        self = cls.from_arrays(st["mst_row"], st["mst_col"], st["delta_crow"], st["delta_col"], st["delta_val"],
                               col_multiplier=st["col_multiplier"])
        self.alpha, self.nnz, self.build_info = st["alpha"], st["nnz"], st["build_info"]
        if st["edge_row"] is not None:
            self._row, self._col = _as_i32(st["edge_row"]), _as_i32(st["edge_col"])
            self._symmetric = None
        return self

    def compression_ratio(self) -> float:
        """Stored elements of the plain CSR (row pointers + columns + values) over stored elements
        of this structure (delta row pointers + columns + values + mst_row + mst_col): the metric
        of benchmark/utility.py:45-64."""
        if self.nnz is None:
            raise RuntimeError("the number of matrix entries is unknown for a structure wrapped from arrays")
        n = self.num_rows
        csr_total = (n + 1) + 2 * self.nnz
        cbm_total = (n + 1) + 2 * int(self._crow[-1]) + self.mst_row.numel() + self.mst_col.numel()
        return csr_total / cbm_total

    # ------------------------------------------------------------------ validation
    def check_format(self, edge_index):
        """Validate the structure against ``edge_index``: walking the tree from the virtual root,
        every row is its parent's column set plus the columns of its positive deltas minus those
        of its negative deltas, and must equal the row of the matrix.  Raises ``ValueError`` with
        the reference's messages (cbm/cbm.py:69-115) on a zero delta or any mismatch.  The matrix
        size is the stored one; the reference derives the root index from ``edge_index[0].max()``
        (cbm/cbm.py:71), which is wrong when the last row is empty."""
        ei = edge_index.detach().cpu().numpy() if isinstance(edge_index, torch.Tensor) else np.asarray(edge_index)
        n = self.num_rows
        if np.any(self._dval == 0):
            raise ValueError(f"Failed with the edge index: {edge_index}")
        # the matrix as sorted unique column arrays per row
        order = np.lexsort((ei[1], ei[0]))
        rows_sorted, cols_sorted = ei[0][order].astype(np.int64), ei[1][order].astype(np.int64)
        keep = np.ones(rows_sorted.shape[0], dtype=bool)
        keep[1:] = (rows_sorted[1:] != rows_sorted[:-1]) | (cols_sorted[1:] != cols_sorted[:-1])
        rows_sorted, cols_sorted = rows_sorted[keep], cols_sorted[keep]
        start = np.searchsorted(rows_sorted, np.arange(n + 1))
        mr, mc = self.mst_row.numpy(), self.mst_col.numpy()
        crow, dcol, dval = self._crow, self._dcol.astype(np.int64), self._dval
        rebuilt: dict[int, np.ndarray] = {n: np.empty(0, dtype=np.int64)}
        pending = deque([n])
        reached = 0
        while pending:
            u = pending.popleft()
            base = rebuilt.pop(u)   # a row's set is only needed until its children are expanded
            for v in mc[mr[u]:mr[u + 1]].tolist():
                d_cols, d_vals = dcol[crow[v]:crow[v + 1]], dval[crow[v]:crow[v + 1]]
                minus = d_cols[d_vals < 0]
                if minus.size and not np.all(np.isin(minus, base)):
                    raise ValueError("Format is incorrect!")   # removes a column the parent does not have
                row_v = np.union1d(np.setdiff1d(base, minus, assume_unique=True), d_cols[d_vals > 0])
                if not np.array_equal(row_v, cols_sorted[start[v]:start[v + 1]]):
                    raise ValueError("Format is incorrect!")
                rebuilt[v] = row_v
                pending.append(v)
                reached += 1
        if reached != n:
            raise ValueError("Format is incorrect!")

    # ------------------------------------------------------------------ plans and dispatch
    def is_symmetric(self) -> bool:
        if self._symmetric is None:
            n = self.num_rows
            a = np.sort(self._row.astype(np.int64) * n + self._col)
            b = np.sort(self._col.astype(np.int64) * n + self._row)
            self._symmetric = bool(np.array_equal(a, b))
        return self._symmetric

    def _device_index(self, t: torch.Tensor | None) -> int:
        if not torch.cuda.is_available():
            raise RuntimeError("cbm4gnn_b200 needs a CUDA device: there is no CPU implementation of the products")
        if t is not None and t.is_cuda:
            return t.device.index if t.device.index is not None else torch.cuda.current_device()
        return torch.cuda.current_device()

    def plan(self, device_index: int | None = None) -> _Plan:
        """The device schedule for one GPU, created on first use and cached."""
        if device_index is None:
            device_index = self._device_index(None)
        p = self._plans.get(device_index)
        if p is None:
            mul = None if self.col_multiplier is None else _as_f32(self.col_multiplier)
            p = _Plan(self.num_rows, self.mst_row.numpy(), self.mst_col.numpy(), self._crow, self._dcol,
                      self._dval, mul, device_index)
            self._plans[device_index] = p
        return p

    def _run(self, fn_name: str, x, y, host_normalized=None):
        L = _lib.lib()
        _check_f32("rhs" if x is not None else "dst", x if x is not None else y)
        _check_f32("dst", y)
        n = self.num_rows
        if y.size(0) != n or (x is not None and (x.size(0) != n or x.size(1) != y.size(1))):
            raise RuntimeError(f"shape mismatch: matrix is {n}x{n}, x {None if x is None else tuple(x.shape)}, "
                               f"y {tuple(y.shape)}")
        f = int(y.size(1))
        if y.is_cuda:
            if x is not None and x.device != y.device:
                raise RuntimeError("x and y must live on the same device")
            p = self.plan(self._device_index(y))
            stream = torch.cuda.current_stream(y.device).cuda_stream
            yp, ldy = _dense_args(y)
            if x is None:
                _lib.check(getattr(L, fn_name)(p.handle, yp, ldy, f, ctypes.c_void_p(stream)))
            else:
                xp, ldx = _dense_args(x)
                _lib.check(getattr(L, fn_name)(p.handle, xp, ldx, yp, ldy, f, ctypes.c_void_p(stream)))
            return
        # CPU tensors, as every caller of the reference passes: stage through the GPU.
        p = self.plan(self._device_index(None))
        if host_normalized is None:
            # update-only and delta-only forms have no host-buffer entry point: stage with torch
            dev = torch.device("cuda", p.device_index)
            yd = y.to(dev)
            self._run(fn_name, None if x is None else x.to(dev), yd)
            y.copy_(yd)
            return
        if not (x.is_contiguous() and y.is_contiguous()):
            raise RuntimeError("host operands must be contiguous")
        _lib.check(L.cbm_b200_spmm_update_host(p.handle, _ptr(x), _ptr(y), f, 1 if host_normalized else 0))

    def _need_multiplier(self):
        if self.col_multiplier is None:
            raise RuntimeError("this cbm_matrix was built with normalized=False: no col_multiplier")

    # ------------------------------------------------------------------ reference method surface
    # "seq_" methods (cbm/cbm.py:144-188) and "omp_" methods (cbm/cbm.py:191-249) share kernels.
    def seq_mkl_csr_spmm_update(self, x, y):
        self._run("cbm_b200_spmm_update", x, y, host_normalized=False)

    def seq_mkl_csr_spmm(self, x, y):
        self._run("cbm_b200_delta_spmm", x, y)

    def seq_mkl_csr_update(self, y):
        self._run("cbm_b200_update", None, y)

    def seq_mkl_csr_fused_spmm_update(self, x, y):
        self._need_multiplier()
        self._run("cbm_b200_fused_spmm_update", x, y, host_normalized=True)

    def seq_mkl_csr_fused_update(self, y):
        self._need_multiplier()
        self._run("cbm_b200_fused_update", None, y)

    omp_mkl_csr_spmm_update = seq_mkl_csr_spmm_update
    omp_mkl_csr_spmm = seq_mkl_csr_spmm
    omp_mkl_csr_update = seq_mkl_csr_update
    omp_avx_csr_update = seq_mkl_csr_update
    omp_mkl_csr_fused_spmm_update = seq_mkl_csr_fused_spmm_update
    omp_mkl_csr_fused_update = seq_mkl_csr_fused_update
    # The reference's omp_mkl_csr_spmm_update_v2 calls a native function that is never exported
    # (cbm/cbm.py:219-228 against cbm/cbm_extensions.cpp:1757-1771) and so always raises; here it
    # is an alias of the working product.
    omp_mkl_csr_spmm_update_v2 = seq_mkl_csr_spmm_update

    # Two-step forms (cbm/cbm.py:255-275): delta product into a new tensor, then the tree update.
    def seq_torch_csr_matmul(self, x):
        y = torch.empty((self.num_rows, x.size(1)), dtype=x.dtype, device=x.device)
        self.seq_mkl_csr_spmm(x, y)
        self.seq_mkl_csr_update(y)
        return y

    def seq_torch_csr_fused_matmul(self, x):
        y = torch.empty((self.num_rows, x.size(1)), dtype=x.dtype, device=x.device)
        self.seq_mkl_csr_spmm(x, y)
        self.seq_mkl_csr_fused_update(y)
        return y

    omp_torch_csr_matmul = seq_torch_csr_matmul
    omp_torch_csr_fused_matmul = seq_torch_csr_fused_matmul

    # ------------------------------------------------------------------ differentiable products
    def transposed(self) -> "cbm_matrix":
        """CBM of the transposed pattern carrying this matrix's multiplier, for gradients of
        non-symmetric graphs.  Symmetric matrices are their own transpose."""
        if self.is_symmetric():
            return self
        if self._transposed is None:
            t = cbm_matrix.__new__(cbm_matrix)
            t.alpha, t.normalized, t.num_rows, t.nnz = self.alpha, self.normalized, self.num_rows, self.nnz
            t.col_multiplier = self.col_multiplier
            mul = None if self.col_multiplier is None else _as_f32(self.col_multiplier)
            order = np.lexsort((self._row, self._col))
            t._row, t._col = np.ascontiguousarray(self._col[order]), np.ascontiguousarray(self._row[order])
            t._build(t._row, t._col, self.num_rows, mul, 0)
            t._symmetric, t._plans, t._transposed = False, {}, self
            t.deltas = None
            self._transposed = t
        return self._transposed

    def matmul(self, x: torch.Tensor, two_step: bool = False) -> torch.Tensor:
        """``A @ x`` (or ``D^-1/2 A D^-1/2 @ x`` when normalized) as a new tensor, differentiable
        with respect to ``x``.  The reference has no gradient for its CBM products (its in-place
        native update is invisible to autograd); the gradient here is the transposed product.
        ``two_step`` runs the forward as the delta product followed by the update-only kernel, the
        path of the reference's ``*_torch_csr_*matmul`` methods (cbm/cbm.py:255-275)."""
        return _CBMMatmul.apply(x, self, two_step)


def _product(cbm: "cbm_matrix", x: torch.Tensor) -> torch.Tensor:
    """``A @ x`` / normalized product into a fresh tensor.  A CUDA operand whose width is not a
    multiple of 4 floats is first copied into a zero-padded buffer: the 128-bit kernel path on
    the padded width is faster than the scalar path on the exact width, copy included."""
    x = x.contiguous()
    f = x.size(1)
    run = cbm.seq_mkl_csr_fused_spmm_update if cbm.normalized else cbm.seq_mkl_csr_spmm_update
    if x.is_cuda and f % 4 != 0 and f > 4:
        fp = -(-f // 4) * 4
        xp = torch.zeros((x.size(0), fp), dtype=x.dtype, device=x.device)
        xp[:, :f] = x
        yp = torch.empty((cbm.num_rows, fp), dtype=x.dtype, device=x.device)
        run(xp, yp)
        return yp[:, :f]
    y = torch.empty((cbm.num_rows, f), dtype=x.dtype, device=x.device)
    run(x, y)
    return y


class _CBMMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cbm, two_step=False):
        ctx.cbm = cbm
        if two_step:
            x = x.contiguous()
            return cbm.seq_torch_csr_fused_matmul(x) if cbm.normalized else cbm.seq_torch_csr_matmul(x)
        return _product(cbm, x)

    @staticmethod
    def backward(ctx, gy):
        return _product(ctx.cbm.transposed(), gy), None, None


class csr_matrix_plan:
    """A plain fp32 CSR matrix resident on one GPU, multiplied by the same kernel as the CBM
    products with every row hanging off the virtual root: the uncompressed comparison of
    benchmark/parallel/benchmark_spmm_cpu.py:112-150 (there MKL's CSR product,
    cbm/cbm_extensions.cpp:1707-1755).  Rows of any length are balanced over the GPU."""

    def __init__(self, crow, col, val, n_cols: int, device_index: int | None = None):
        crow, col, val = _as_i32(crow), _as_i32(col), _as_f32(val)
        self.n_rows, self.n_cols = crow.shape[0] - 1, int(n_cols)
        if device_index is None:
            device_index = torch.cuda.current_device()
        self.device_index = device_index
        self.handle = ctypes.c_void_p(0)
        _lib.check(_lib.lib().cbm_b200_csr_plan_create(self.n_rows, self.n_cols, _ptr(crow), _ptr(col), _ptr(val),
                                                       device_index, ctypes.byref(self.handle)))

    def matmul(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        _check_f32("rhs", x)
        if x.size(0) != self.n_cols:
            raise RuntimeError(f"shape mismatch: matrix is {self.n_rows}x{self.n_cols}, x {tuple(x.shape)}")
        y = out if out is not None else torch.empty((self.n_rows, x.size(1)), dtype=x.dtype, device=x.device)
        xp, ldx = _dense_args(x)
        yp, ldy = _dense_args(y)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(_lib.lib().cbm_b200_spmm_update(self.handle, xp, ldx, yp, ldy, int(x.size(1)), ctypes.c_void_p(stream)))
        return y

    def status(self, stream=0):
        _lib.check(_lib.lib().cbm_b200_plan_status(self.handle, ctypes.c_void_p(stream)))

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().cbm_b200_plan_destroy(self.handle)
                self.handle = ctypes.c_void_p(0)
        except Exception:
            pass
