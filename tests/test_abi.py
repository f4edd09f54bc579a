"""The C ABI: the library loads without a GPU and exports exactly what include/cbm_b200.h declares."""
import ctypes
import os
import re

import pytest

from cbm4gnn_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "cbm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cbm_b200_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    L = _lib.lib()
    names = _declared()
    assert len(names) >= 19
    for name in names:
        assert hasattr(L, name), name
    assert sorted(_lib.EXPORTED) == names


def test_version_and_error_slot():
    L = _lib.lib()
    assert L.cbm_b200_version().startswith(b"cbm_b200")
    assert L.cbm_b200_built_info(None, None, None, None, None, None) == 1
    assert b"NULL" in L.cbm_b200_last_error()
    with pytest.raises(RuntimeError, match="cbm_b200 error 1"):
        _lib.check(1)


def test_null_plan_arguments_are_rejected_without_a_gpu():
    L = _lib.lib()
    assert L.cbm_b200_plan_info(None, None, None, None, None, None) == 1
    assert L.cbm_b200_spmm_update(None, None, 0, None, 0, 4, None) == 1
    assert L.cbm_b200_plan_create(4, None, None, None, None, None, None, None, 0, 0, 4, 0,
                                  ctypes.byref(ctypes.c_void_p(0))) == 1
    L.cbm_b200_plan_destroy(None)


def test_products_fail_loudly_without_cuda():
    import numpy as np
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from cbm4gnn_b200.cbm import cbm_matrix
    from cbm4gnn_b200 import graphs
    ei = torch.from_numpy(graphs.erdos_renyi(10, 0.5, 0)).to(torch.int32)
    c = cbm_matrix(ei, torch.ones(ei.shape[1]))
    x = torch.ones((c.num_rows, 4))
    with pytest.raises(RuntimeError, match="CUDA"):
        c.seq_torch_csr_matmul(x)
