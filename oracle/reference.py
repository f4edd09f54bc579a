"""TEST INFRASTRUCTURE — access to the reference's own code.

``ref_module()`` loads ``oracle/_ref/cbm_mkl_cpp.so``: the reference's unmodified
cbm/cbm_extensions.cpp compiled by ``oracle/build_ref.py`` (pybind11 module with the 13 functions of
cbm/cbm_extensions.cpp:1757-1771).  The prebuilt file is all that is needed at run time.

``reference_cbm_class()`` additionally imports the reference's unmodified Python class
(cbm/cbm.py) on top of that module; it needs the reference checkout and is used only by the script
that generates the committed fixtures.

Only tests, the smoke check and bench.py's CPU legs may import this file.
"""
from __future__ import annotations

import importlib.util
import os
import sys

from . import build_ref

_mod = None


def ref_available() -> bool:
    return os.path.exists(build_ref.OUT)


def ref_module():
    """The reference's native module, or RuntimeError when it has not been built."""
    global _mod
    if _mod is None:
        if not ref_available():
            raise RuntimeError("oracle/_ref/cbm_mkl_cpp.so is missing: run python oracle/build_ref.py "
                               "where the reference sources are present")
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        spec = importlib.util.spec_from_file_location("cbm_mkl_cpp", build_ref.OUT)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    return _mod


def reference_cbm_class(ref_dir: str = build_ref.DEFAULT_REFERENCE):
    """``cbm_matrix`` of the reference's cbm/cbm.py, imported unmodified with its native module
    name ``cbm.cbm_mkl_cpp`` bound to ``oracle/_ref``."""
    if not os.path.exists(os.path.join(ref_dir, "cbm", "cbm.py")):
        raise RuntimeError("reference checkout not found at " + ref_dir)
    mod = ref_module()
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import cbm  # namespace package: the reference's cbm/ directory
    sys.modules["cbm.cbm_mkl_cpp"] = mod
    cbm.cbm_mkl_cpp = mod
    from cbm.cbm import cbm_matrix
    return cbm_matrix


def threads(n: int) -> None:
    """Thread count for both halves of the reference's parallel path: the oneMKL inside libtorch
    and the OpenMP team of its tree update."""
    import torch
    torch.set_num_threads(n)
