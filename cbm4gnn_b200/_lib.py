"""Builds and loads ``libcbm_b200.so`` and declares its C ABI for ``ctypes``.

The shared library is the only native module of the package.  It takes the place of the pybind11
module ``cbm.cbm_mkl_cpp`` of the reference (cbm/cbm_extensions.cpp:1757-1771, built by
cbm/setup.py:15-47 against MKL and arbok); it is compiled in-tree with ``nvcc`` for sm_100a and has
no dependency besides the CUDA runtime and libgomp.

There is deliberately no CPU fallback: if the library is missing or fails to load, every product
entry point of the package raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from ctypes import POINTER, c_char_p, c_double, c_float, c_int32, c_int64, c_void_p

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG_DIR)
LIB_PATH = os.path.join(_PKG_DIR, "libcbm_b200.so")
SOURCES = [
    os.path.join(_PKG_DIR, "csrc", "cbm_engine.cu"),
    os.path.join(_PKG_DIR, "csrc", "cbm_builder.cpp"),
    os.path.join(_PKG_DIR, "csrc", "cbm_dense.cu"),
    os.path.join(_PKG_DIR, "csrc", "cbm_dense_grad.cu"),
    os.path.join(_PKG_DIR, "csrc", "cbm_candidates.cu"),
]
HEADERS = [
    os.path.join(_ROOT, "include", "cbm_b200.h"),
    os.path.join(_PKG_DIR, "csrc", "cbm_common.h"),
    os.path.join(_PKG_DIR, "csrc", "cbm_candidates.h"),
    os.path.join(_PKG_DIR, "csrc", "cbm_dense_gemm.cuh"),
]
_OBJ_DIR = os.path.join(_PKG_DIR, "build")


def _cutlass_includes() -> list[str]:
    """Header trees of CUTLASS / CuTe (the dense maps instantiate their sm100 templates): the
    environment variable CUTLASS_HOME, else the copy vendored inside the flashinfer package."""
    roots = [os.environ.get("CUTLASS_HOME")]
    try:
        import importlib.util
        spec = importlib.util.find_spec("flashinfer")
        if spec and spec.submodule_search_locations:
            roots.append(os.path.join(list(spec.submodule_search_locations)[0], "data", "cutlass"))
    except Exception:
        pass
    for r in roots:
        if r and os.path.exists(os.path.join(r, "include", "cutlass", "cutlass.h")):
            return [os.path.join(r, "include"), os.path.join(r, "tools", "util", "include")]
    raise RuntimeError("CUTLASS headers not found: set CUTLASS_HOME (needed to compile csrc/cbm_dense.cu)")

# Every symbol include/cbm_b200.h declares; the CPU test-suite checks the library exports all of them.
EXPORTED = [
    "cbm_b200_last_error",
    "cbm_b200_version",
    "cbm_b200_build",
    "cbm_b200_build_gpu",
    "cbm_b200_built_candidates_on_gpu",
    "cbm_b200_built_info",
    "cbm_b200_built_export_csr",
    "cbm_b200_built_export_coo",
    "cbm_b200_built_free",
    "cbm_b200_plan_create",
    "cbm_b200_plan_destroy",
    "cbm_b200_schedule_info",
    "cbm_b200_plan_info",
    "cbm_b200_plan_tune",
    "cbm_b200_plan_status",
    "cbm_b200_spmm_update",
    "cbm_b200_fused_spmm_update",
    "cbm_b200_update",
    "cbm_b200_fused_update",
    "cbm_b200_delta_spmm",
    "cbm_b200_csr_spmm",
    "cbm_b200_csr_plan_create",
    "cbm_b200_spmm_update_bcast",
    "cbm_b200_probe_l2_read_gbps",
    "cbm_b200_dense_forward",
    "cbm_b200_dense_forward_relu",
    "cbm_b200_dense_grad_input",
    "cbm_b200_dense_grad_input_relu",
    "cbm_b200_dense_grad_weight",
    "cbm_b200_dense_grad_weight_workspace",
    "cbm_b200_spmm_update_host",
    "cbm_b200_copy2d_async",
    "cbm_b200_spmm_update_static",
    "cbm_b200_selftest_wait",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: cannot build libcbm_b200.so")


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library for sm_100a next to this file and return its path.  Every source is
    compiled to its own object (kept under ``build/``, so that touching the engine does not
    recompile the CUTLASS instantiations, which take over a minute) and the objects are linked."""
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(_OBJ_DIR, exist_ok=True)
    newest_header = max(os.path.getmtime(h) for h in HEADERS)
    objs, jobs = [], []
    for src in SOURCES:
        obj = os.path.join(_OBJ_DIR, os.path.splitext(os.path.basename(src))[0] + ".o")
        objs.append(obj)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), newest_header):
            continue
        cmd = [
            _nvcc(), "-O3", "-std=c++17",
            "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
            "-Xcompiler", "-fPIC,-fopenmp,-O3",
            "-I", os.path.join(_ROOT, "include"),
            "-I", os.path.join(_PKG_DIR, "csrc"),
        ]
        if os.path.basename(src).startswith("cbm_dense"):
            cmd += ["--expt-relaxed-constexpr", "-diag-suppress", "20012"]
            for inc in _cutlass_includes():
                cmd += ["-I", inc]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        cmd += ["-c", src, "-o", obj]
        jobs.append(cmd)

    def compile_one(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
        return res.stderr

    # the sources are compiled side by side: the CUTLASS instantiations alone take minutes
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=max(1, len(jobs))) as pool:
        log = list(pool.map(compile_one, jobs))
    cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs, "-lgomp"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print("".join(log))
    return LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library (built on first use when the sources are newer than the binary)."""
    global _lib
    if _lib is not None:
        return _lib
    if needs_build():
        build()
    L = ctypes.CDLL(LIB_PATH)
    i32p, f32p = POINTER(c_int32), POINTER(c_float)

    def sig(name, restype, *argtypes):
        fn = getattr(L, name)
        fn.restype = restype
        fn.argtypes = list(argtypes)

    sig("cbm_b200_last_error", c_char_p)
    sig("cbm_b200_version", c_char_p)
    sig("cbm_b200_build", c_int32, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_void_p, c_int32,
        POINTER(c_void_p))
    sig("cbm_b200_build_gpu", c_int32, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_void_p, c_int32, c_int32,
        POINTER(c_void_p))
    sig("cbm_b200_built_candidates_on_gpu", c_int32, c_void_p)
    sig("cbm_b200_built_info", c_int32, c_void_p, POINTER(c_int64), POINTER(c_int64), i32p, i32p,
        POINTER(c_double))
    sig("cbm_b200_built_export_csr", c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p)
    sig("cbm_b200_built_export_coo", c_int32, c_void_p, c_void_p, c_void_p, c_void_p)
    sig("cbm_b200_built_free", None, c_void_p)
    sig("cbm_b200_plan_create", c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, POINTER(c_void_p))
    sig("cbm_b200_plan_destroy", None, c_void_p)
    sig("cbm_b200_schedule_info", c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_int32, c_int32, c_int32, i32p, i32p, i32p, i32p)
    sig("cbm_b200_plan_info", c_int32, c_void_p, i32p, POINTER(c_int64), i32p, i32p,
        POINTER(c_int64))
    sig("cbm_b200_plan_tune", c_int32, c_void_p, c_int32, c_int32, c_int32, c_int32)
    sig("cbm_b200_plan_status", c_int32, c_void_p, c_void_p)
    for name in ("cbm_b200_spmm_update", "cbm_b200_fused_spmm_update", "cbm_b200_delta_spmm"):
        sig(name, c_int32, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int32, c_void_p)
    for name in ("cbm_b200_update", "cbm_b200_fused_update"):
        sig(name, c_int32, c_void_p, c_void_p, c_int64, c_int32, c_void_p)
    sig("cbm_b200_csr_spmm", c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_int64, c_void_p, c_int64, c_int32, c_void_p)
    sig("cbm_b200_csr_plan_create", c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int32,
        POINTER(c_void_p))
    sig("cbm_b200_spmm_update_bcast", c_int32, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32,
        c_int32, c_int32, POINTER(c_void_p), c_void_p)
    sig("cbm_b200_probe_l2_read_gbps", c_double, c_int32)
    for name in ("cbm_b200_dense_forward", "cbm_b200_dense_forward_relu", "cbm_b200_dense_grad_input"):
        sig(name, c_int32, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32, c_void_p)
    sig("cbm_b200_dense_grad_input_relu", c_int32, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
        c_int32, c_int32, c_int32, c_void_p)
    sig("cbm_b200_dense_grad_weight", c_int32, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int32,
        c_int32, c_int32, c_void_p, c_int64, c_void_p)
    sig("cbm_b200_dense_grad_weight_workspace", c_int64, c_int32, c_int32, c_int32)
    sig("cbm_b200_copy2d_async", c_int32, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p)
    sig("cbm_b200_spmm_update_host", c_int32, c_void_p, c_void_p, c_void_p, c_int32, c_int32)
    sig("cbm_b200_spmm_update_static", c_int32, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int32,
        c_int32, c_void_p)
    sig("cbm_b200_selftest_wait", c_int32, c_int32, c_int32, c_void_p)
    _lib = L
    return L


def check(status: int) -> None:
    """Raise ``RuntimeError`` carrying the library's message for a non-zero status.

    The reference turns dtype errors into ``RuntimeError`` through ``TORCH_CHECK``
    (cbm/cbm_extensions.cpp:659-666) and kills the process on MKL errors (cbm/helpers.hpp:57-85);
    here every native failure surfaces as ``RuntimeError``.
    """
    if status != 0:
        msg = lib().cbm_b200_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"cbm_b200 error {status}: {msg}")
