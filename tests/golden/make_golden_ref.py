"""Generates ``cbm_reference.npz``: outputs of the REFERENCE ITSELF on small seeded inputs.

Every array in the file was produced by the reference's unmodified Python class (cbm/cbm.py) on top
of its unmodified native source (cbm/cbm_extensions.cpp) compiled into ``oracle/_ref`` by
``oracle/build_ref.py`` — the sparse product inside is Intel oneMKL's (the copy libtorch ships), the
tree updates are the reference's compiled loops, the structure comes out of the reference's
``cbm_init_v1_/v2_`` (with the stand-in ``A * A^T`` and arborescence solver of ``oracle/ref_shim``).

Shapes follow the reference's own tests: Erdős–Rényi graphs with 25 nodes, p = 0.5 / 0.75, F = 10,
integer-valued features, alpha = 3 (tests/test_matmul_correctness.py:11-61), plus a 40- and a
64-node graph with Gaussian features and widths 7 and 47, and a 300-node copy-model graph whose tree
is several levels deep.  For each case and for both the plain and the normalized form the file holds
the structure (``mst_row``, ``mst_col``, delta CSR, ``col_multiplier``) and the result of every
product method of the reference (cbm/cbm.py:144-275).

Needs the reference checkout; run from the repository root:
    python oracle/build_ref.py && python tests/golden/make_golden_ref.py
"""
import contextlib
import io
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..")
sys.path.insert(0, ROOT)
from cbm4gnn_b200 import graphs  # noqa: E402
from oracle import reference  # noqa: E402

CASES = [
    # name, graph, features, alpha
    ("er25a", ("er", 25, 0.5, 7000), ("int", 10, 8000), 3),
    ("er25b", ("er", 25, 0.75, 7001), ("int", 10, 8001), 3),
    ("er40", ("er", 40, 0.3, 7002), ("normal", 7, 8002), 1),
    ("er64", ("er", 64, 0.2, 7003), ("normal", 47, 8003), 0),
    ("copy300", ("copy", 300, 0.8, 7004), ("normal", 36, 8004), 2),
]


def make_inputs(graph, feats):
    kind = graph[0]
    if kind == "er":
        ei = graphs.erdos_renyi(graph[1], graph[2], graph[3])
    else:
        ei = graphs.copy_model(graph[1], graph[2], 3, graph[3], None)
    order = np.lexsort((ei[1], ei[0]))  # (row, col) sorted, as torch_geometric hands edge lists over
    ei = np.ascontiguousarray(ei[:, order])
    n = int(ei.max()) + 1
    rng = np.random.default_rng(feats[2])
    if feats[0] == "int":
        x = rng.integers(0, 10, size=(n, feats[1])).astype(np.float32)
    else:
        x = rng.standard_normal((n, feats[1])).astype(np.float32)
    return ei, x


def run_reference(cbm_matrix, ei, x, alpha, normalized):
    e = torch.from_numpy(ei).to(torch.int32)
    if normalized:
        n = int(ei.max()) + 1
        loops = torch.arange(n, dtype=torch.int32)
        e = torch.cat([e, torch.stack([loops, loops])], dim=1)
        order = np.lexsort((e[1].numpy(), e[0].numpy()))
        e = e[:, order].contiguous()
    values = torch.ones(e.size(1), dtype=torch.float32)
    with contextlib.redirect_stdout(io.StringIO()):
        c = cbm_matrix(e, values, alpha=alpha, normalized=normalized)
    xt = torch.from_numpy(x)
    out = dict(edge_index=e.numpy(), mst_row=c.mst_row.numpy(), mst_col=c.mst_col.numpy(),
               crow=c.deltas.crow_indices().numpy().astype(np.int32),
               col=c.deltas.col_indices().numpy().astype(np.int32), val=c.deltas.values().numpy())
    assert tuple(c.deltas.shape) == (x.shape[0], x.shape[0]), "delta tensor smaller than the matrix"
    with contextlib.redirect_stdout(io.StringIO()):
        c.check_format(e)

    def two(name):  # in-place (x, y) forms
        y = torch.zeros_like(xt)
        getattr(c, name)(xt, y)
        return y.numpy()

    def upd(name):  # update-only forms on y = deltas @ x
        y = (c.deltas @ xt).contiguous()
        getattr(c, name)(y)
        return y.numpy()

    out["delta_x"] = (c.deltas @ xt).numpy()
    out["seq_mkl_csr_spmm"] = two("seq_mkl_csr_spmm")
    out["omp_mkl_csr_spmm"] = two("omp_mkl_csr_spmm")
    if not normalized:
        out["seq_mkl_csr_spmm_update"] = two("seq_mkl_csr_spmm_update")
        out["omp_mkl_csr_spmm_update"] = two("omp_mkl_csr_spmm_update")
        out["seq_mkl_csr_update"] = upd("seq_mkl_csr_update")
        out["omp_mkl_csr_update"] = upd("omp_mkl_csr_update")
        if x.shape[1] % 32 == 0 or x.shape[1] < 16:
            # the AVX form mis-steps its column loop for other widths (i += 15 at
            # cbm/cbm_extensions.cpp:1683); those widths are left out
            out["omp_avx_csr_update"] = upd("omp_avx_csr_update")
        out["seq_torch_csr_matmul"] = c.seq_torch_csr_matmul(xt).numpy()
        out["omp_torch_csr_matmul"] = c.omp_torch_csr_matmul(xt).numpy()
    else:
        out["col_multiplier"] = c.col_multiplier.numpy()
        out["seq_mkl_csr_fused_spmm_update"] = two("seq_mkl_csr_fused_spmm_update")
        out["omp_mkl_csr_fused_spmm_update"] = two("omp_mkl_csr_fused_spmm_update")
        out["seq_mkl_csr_fused_update"] = upd("seq_mkl_csr_fused_update")
        out["omp_mkl_csr_fused_update"] = upd("omp_mkl_csr_fused_update")
        out["seq_torch_csr_fused_matmul"] = c.seq_torch_csr_fused_matmul(xt).numpy()
        # omp_torch_csr_fused_matmul has no return statement (cbm/cbm.py:272-274): nothing to record
    return out


def main():
    cbm_matrix = reference.reference_cbm_class()
    torch.set_num_threads(4)
    blob = {"names": np.array([c[0] for c in CASES])}
    for name, graph, feats, alpha in CASES:
        ei, x = make_inputs(graph, feats)
        blob[f"{name}/x"] = x
        blob[f"{name}/alpha"] = np.array(alpha)
        for normalized in (False, True):
            tag = "norm" if normalized else "plain"
            for k, v in run_reference(cbm_matrix, ei, x, alpha, normalized).items():
                blob[f"{name}/{tag}/{k}"] = v
    # many methods return bit-identical arrays (seq_ and omp_ forms, one-step and two-step forms):
    # each distinct array is stored once, "aliases" maps the other keys to the stored one
    stored, first_key, aliases = {}, {}, {}
    for k, v in blob.items():
        sig = (v.dtype.str, v.shape, v.tobytes())
        if sig in first_key:
            aliases[k] = first_key[sig]
        else:
            first_key[sig] = k
            stored[k] = v
    stored["aliases"] = np.array(json.dumps(aliases))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cbm_reference.npz")
    np.savez_compressed(path, **stored)
    print("wrote", path, os.path.getsize(path), "bytes,", len(blob), "arrays,", len(aliases), "of them aliases")


if __name__ == "__main__":
    main()
