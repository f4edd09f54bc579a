"""cbm4gnn_b200 — compressed-binary-matrix (CBM) sparse products and GCN layers on NVIDIA B200.

Drop-in for the CBM path of cbm4scale/cbm4gnn: ``cbm_matrix`` keeps the reference's constructor and
method names (cbm/cbm.py), the products run as hand-written sm_100a CUDA kernels reached through
the C ABI of ``libcbm_b200.so`` (include/cbm_b200.h).
"""
from .cbm import cbm_matrix  # noqa: F401

__all__ = ["cbm_matrix"]
