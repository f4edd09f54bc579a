"""Choice of the ``alpha`` threshold for a graph.

The reference sweeps alpha over {0, 1, 2, 4, ..., 128} for several operand widths and keeps a hand
table per dataset (alpha_searcher/spmm_cpu_parallel.py:16-18, 44-168; the table itself at
benchmark/parallel/benchmark_gcn_cpu.py:44-56).  ``search_alpha`` does the sweep for one graph:
every candidate alpha is built once, and candidates are ranked either by the measured time of the
CUDA product (median of ``iters`` launches, the reference's statistic) or, without a GPU, by the
bytes the product has to move — delta entries times operand width dominates, so the byte model
orders candidates the way time does on a memory-bound kernel.
"""
from __future__ import annotations

import numpy as np
import torch

from .cbm import cbm_matrix

DEFAULT_ALPHAS = (0, 1, 2, 4, 8, 16, 32, 64)


def product_bytes(n_rows: int, n_delta: int, n_root_children: int, f: int) -> int:
    """Bytes one product must move: delta row pointers and indices, one gathered operand row per
    delta entry, one parent row per row below the first level, the output, and the per-row
    parent/scale words."""
    return (4 * (n_rows + 1) + 4 * n_delta + 4 * f * n_delta + 4 * f * (n_rows - n_root_children)
            + 4 * f * n_rows + 8 * n_rows)


def search_alpha(edge_index, f: int, alphas=DEFAULT_ALPHAS, normalized: bool = False, measure: bool | None = None,
                 iters: int = 50, device=None):
    """Build the structure for every alpha and rank them.

    Returns ``(best_alpha, table)`` where ``table`` has one dict per alpha with ``alpha``,
    ``n_delta``, ``n_root_children``, ``depth``, ``compression_ratio``, ``build_seconds``,
    ``bytes`` and, when measured, ``ms``.  ``measure=None`` measures iff CUDA is available.
    """
    ei = edge_index if isinstance(edge_index, torch.Tensor) else torch.as_tensor(edge_index)
    values = torch.ones(ei.size(1))
    if measure is None:
        measure = torch.cuda.is_available()
    if measure and not torch.cuda.is_available():
        raise RuntimeError("measure=True needs a CUDA device")
    table = []
    x = y = None
    for alpha in alphas:
        c = cbm_matrix(ei.to(torch.int32), values, alpha=int(alpha), normalized=normalized,
                       build_device=torch.cuda.current_device() if measure else None)
        info = c.build_info
        row = dict(alpha=int(alpha), n_delta=info["n_delta"], n_root_children=info["n_root_children"],
                   depth=info["depth"], compression_ratio=c.compression_ratio(),
                   build_seconds=info["seconds_total"],
                   bytes=product_bytes(c.num_rows, info["n_delta"], info["n_root_children"], f))
        if measure:
            dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
            if x is None:
                x = torch.randn((c.num_rows, f), device=dev)
                y = torch.empty_like(x)
            run = c.omp_mkl_csr_fused_spmm_update if normalized else c.omp_mkl_csr_spmm_update
            run(x, y)  # plan creation and first launch outside the timing
            times = []
            for _ in range(iters):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                run(x, y)
                e1.record()
                e1.synchronize()
                times.append(e0.elapsed_time(e1))
            row["ms"] = float(np.median(times))
        table.append(row)
    key = "ms" if measure else "bytes"
    best = min(table, key=lambda r: (r[key], r["alpha"]))
    return best["alpha"], table
