"""TEST INFRASTRUCTURE — compiles the reference's own native module, unmodified, into ``oracle/_ref``.

``cbm/cbm_extensions.cpp`` of the reference is compiled from where it lies (nothing is copied) with
the include path pointed at ``oracle/ref_shim``: stand-in ``mkl.h`` / ``mkl_spblas.h`` /
``arbok/tarjan/tarjan_pq.h`` for the two dependencies that are not installed offline.  The
stand-ins forward the compute path's sparse product to the real oneMKL routines that
``libtorch_cpu.so`` exports, so what comes out is the reference's pybind11 module ``cbm_mkl_cpp``
(cbm/cbm_extensions.cpp:1757-1771) with all 13 functions: its tree updates are the reference's
compiled source, its ``deltas * rhs`` is Intel's, its builder is the reference's candidate / BFS /
delta code over a substituted ``A * A^T`` and arborescence solver.

    python oracle/build_ref.py [--reference DIR] [--force]

The output ``oracle/_ref/cbm_mkl_cpp.so`` is git-ignored and is loaded only by the tests, the smoke
check and bench.py's CPU legs (``oracle.ref_module()``).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

_DIR = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(_DIR, "_ref")
OUT = os.path.join(OUT_DIR, "cbm_mkl_cpp.so")
SHIM = os.path.join(_DIR, "ref_shim")
DEFAULT_REFERENCE = os.environ.get("CBM_REFERENCE_DIR", "/root/reference")


def reference_source(ref_dir: str = DEFAULT_REFERENCE) -> str | None:
    src = os.path.join(ref_dir, "cbm", "cbm_extensions.cpp")
    return src if os.path.exists(src) else None


def build(ref_dir: str = DEFAULT_REFERENCE, force: bool = False, verbose: bool = False) -> str | None:
    """Returns the path of the built module, or None when the reference sources are not present
    (then an existing ``oracle/_ref`` is used as it is)."""
    src = reference_source(ref_dir)
    if src is None:
        return OUT if os.path.exists(OUT) else None
    deps = [src, os.path.join(ref_dir, "cbm", "helpers.hpp"), os.path.join(SHIM, "ref_shim.cpp"),
            os.path.join(SHIM, "mkl.h"), os.path.join(SHIM, "mkl_spblas.h"),
            os.path.join(SHIM, "arbok", "tarjan", "tarjan_pq.h")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(d) <= os.path.getmtime(OUT) for d in deps):
        return OUT
    import torch
    from torch.utils import cpp_extension
    os.makedirs(OUT_DIR, exist_ok=True)
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++20", "-fopenmp", "-mavx2", "-mfma", "-fPIC", "-shared", "-w",
           "-DTORCH_EXTENSION_NAME=cbm_mkl_cpp", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
           "-I", SHIM, "-I", os.path.join(ref_dir, "cbm")]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += ["-isystem", sysconfig.get_paths()["include"]]
    cmd += [src, os.path.join(SHIM, "ref_shim.cpp"), "-o", OUT,
            "-L", tlib, "-Wl,-rpath," + tlib, "-ltorch_python", "-ltorch", "-ltorch_cpu", "-lc10", "-lgomp"]
    if verbose:
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("building oracle/_ref failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(a.reference, force=a.force, verbose=True)
    print(out or "reference sources not found and no prebuilt oracle/_ref")
    sys.exit(0 if out else 1)
