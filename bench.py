#!/usr/bin/env python
"""Benchmark of the CBM product on B200: one step = one normalized product
``Y = D^-1/2 (A+I) D^-1/2 X`` over the whole synthetic operand.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2]

Workload (N = 1): copy-model graph, 100 000 nodes, p_copy = 0.7, 5 random links, degree cap 5 000,
self loops added, alpha = 8, X = 100 000 x 500 fp32 N(0,1) — synthetic stand-in with the shape of
the second benchmark configuration.  With N > 1 the graph has N x 100 000 nodes (same generator:
weak scaling), its root subtrees are partitioned over the ranks, every rank holds all of X and
computes its shard; the product itself needs no exchange, so none is timed.

The JSON line reports, for the timed region, the algorithmic bytes the product must move
(delta row pointers + delta indices + one gathered operand row per delta entry + one parent row
per non-root row + Y written once + per-row parent/scale words) divided by time.

``--impl reference`` times the reference's own CPU path for the same product on the host cores:
``y = deltas @ x`` through torch's CSR kernel (MKL inside libtorch, the path of cbm/cbm.py:271-275)
followed by the restated OpenMP tree update.  The reference's native module itself cannot be built
offline (needs oneMKL headers and the arbok submodule).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the product kernel, from the ncu
# captures summarised under profiles/ (key: workload, operand width, GPUs, scale).
DRAM_TRAFFIC: dict = {
    ("c2", 500, 1, 1.0): 2.078e9,  # profiles/cbm_items_kernel_c2_f500.md
    ("c4", 128, 1, 1.0): 1.238e9,  # profiles/cbm_items_kernel_c4_f128.md
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="with N > 1: weak = graph grows with N (default), strong = same graph sharded")
    ap.add_argument("--task", default="spmm", choices=["spmm", "gcn", "build", "csr"],
                    help="spmm: one CBM product per step (the headline); gcn: forward+backward of the "
                         "stacked GCN of the workload, reported in ms; build: host builder time and "
                         "compression ratio over alpha in {0,1,2,4,...,64} (no GPU needed); csr: the "
                         "uncompressed comparison — plain CSR product of the same (normalized) matrix")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the graph (profiling captures)")
    ap.add_argument("--f", type=int, default=0, help="override the operand width")
    ap.add_argument("--alpha", type=int, default=-1, help="override the workload's alpha")
    ap.add_argument("--slab", type=int, default=0)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--host-chunk", type=int, default=0)
    ap.add_argument("--form", type=int, default=0, help="0 register form (default), 1 bulk-copy form")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    return ap.parse_args()


def algorithmic_bytes(n_rows, n_delta, n_root_children, f, normalized=True):
    """Bytes one product must move: 4(N+1) row pointers + 4 nnzD indices + 4 F nnzD gathered rows
    + 4 F (N - roots) parent rows + 4 F N output + 8 N parent/scale words."""
    from cbm4gnn_b200.alpha_search import product_bytes
    return product_bytes(n_rows, n_delta, n_root_children, f)


def make_workload(args, world):
    import torch
    if args.scaling == "strong":
        world = 1
    from cbm4gnn_b200 import graphs
    from cbm4gnn_b200.cbm import cbm_matrix
    from cbm4gnn_b200.utility import add_self_loops
    cfg = dict(graphs.CONFIGS[args.workload])
    if args.alpha >= 0:
        cfg["alpha"] = args.alpha
    t0 = time.time()
    if cfg["kind"] == "copy":
        n = max(64, int(cfg["n"] * args.scale)) * world
        ei = graphs.copy_model(n, cfg["p_copy"], cfg["n_random"], cfg["seed"], cfg["max_degree"])
    else:
        ei = graphs.make_graph(args.workload, scale=args.scale * world)
    e = torch.from_numpy(ei)
    if cfg["normalized"]:
        e = add_self_loops(e)
    t1 = time.time()
    # torchrun pins OMP_NUM_THREADS to 1; the host builder gets its share of the cores explicitly
    ranks_here = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
    c = cbm_matrix(e.to(torch.int32), torch.ones(e.shape[1]), alpha=cfg["alpha"], normalized=cfg["normalized"],
                   n_threads=max(1, (os.cpu_count() or 1) // max(1, ranks_here)))
    f = args.f or cfg["f"]
    x = graphs.make_features(args.workload, c.num_rows, f=f)
    info = dict(workload=args.workload, n=c.num_rows, nnz=int(e.shape[1]), f=f, alpha=cfg["alpha"],
                normalized=cfg["normalized"], n_delta=c.build_info["n_delta"],
                n_root_children=c.build_info["n_root_children"], depth=c.build_info["depth"],
                graph_seconds=round(t1 - t0, 2), build_seconds=round(c.build_info["seconds_total"], 3))
    return c, x, info


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, util, reasons, mx = [], [], set(), None
        try:
            for line in open(self.path):
                p = [t.strip() for t in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    mx = float(p[2])
                    util.append(float(p[9]) if len(p) > 9 else 0.0)
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            busy = [v for v, u in zip(sm, util) if u > 0] or sm
            out = dict(sm_mhz=float(np.median(busy)), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm),
                       samples_under_load=len([u for u in util if u > 0]))
        return out


def cpu_reference(c, x, seconds, threads=None, steps=None, warmup=1):
    """The reference's CPU path (cbm/cbm.py:271-275) on the host: torch CSR product (MKL) + OpenMP
    tree update.  Either exactly ``steps`` products after ``warmup``, or (steps None) repeated for
    about ``seconds`` after one warm-up; returns seconds per product, products timed, threads."""
    import torch
    from oracle import cbm_oracle as orc
    threads = threads or os.cpu_count()
    torch.set_num_threads(threads)
    orc.clib().oracle_set_threads(threads)
    xt = torch.from_numpy(x)
    mr, mc = c.mst_row.numpy(), c.mst_col.numpy()
    mult = None if c.col_multiplier is None else c.col_multiplier.numpy()

    def once():
        y = (c.deltas @ xt).numpy()
        if mult is None:
            orc.update(mr, mc, y, parallel=True)
        else:
            orc.fused_update(mr, mc, mult, y, parallel=True)
        return y

    for _ in range(max(1, warmup)):
        once()
    t0 = time.perf_counter()
    it = 0
    while True:
        once()
        it += 1
        el = time.perf_counter() - t0
        if (steps is not None and it >= steps) or (steps is None and (el > seconds or it >= 50)):
            break
    return el / it, it, threads


def gcn_task(args):
    """Forward + backward of the workload's GCN stack (widths from the configuration, ReLU between
    layers, loss = sum of outputs) on one GPU; prints one JSON line with ms per step and the split
    between CBM products and everything else."""
    import torch
    from cbm4gnn_b200 import graphs
    from cbm4gnn_b200.gcn import GCNModel
    cfg = graphs.CONFIGS[args.workload]
    widths = cfg.get("widths", (cfg["f"], 256, 64))
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return sharded_gcn_task(args, widths)
    c, x, info = make_workload(args, 1)
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    model = GCNModel(widths, structure=c, alpha=cfg["alpha"]).to(dev)
    xd = torch.from_numpy(x).to(dev).requires_grad_(True)
    ei = torch.zeros((2, 1), dtype=torch.int64)  # the shared structure is already cached in every layer
    train = len(widths) == 3

    def step():
        if train:
            model.zero_grad(set_to_none=True)
            xd.grad = None
            model(xd, ei).sum().backward()
        else:
            with torch.no_grad():
                model(xd, ei)

    for _ in range(max(3, args.warmup)):
        step()
    c.plan(0).status()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    # the CBM products alone, same operand widths (forward, and backward when training)
    plan, L = c.plan(0), None
    from cbm4gnn_b200 import _lib
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    prod_ms = 0.0
    for f in list(widths[1:]) * (2 if train else 1):
        a = torch.randn((c.num_rows, f), device=dev)
        b = torch.empty_like(a)
        for _ in range(3):
            _lib.check(L.cbm_b200_fused_spmm_update(plan.handle, a.data_ptr(), f, b.data_ptr(), f, f, st))
        e0.record()
        for _ in range(10):
            _lib.check(L.cbm_b200_fused_spmm_update(plan.handle, a.data_ptr(), f, b.data_ptr(), f, f, st))
        e1.record()
        torch.cuda.synchronize()
        prod_ms += e0.elapsed_time(e1) / 10
    print(json.dumps(dict(metric="gcn_%dlayer_%s_ms" % (len(widths) - 1, "fwd_bwd" if train else "fwd"), value=ms,
                          unit="ms", n_gpus=1, steps=args.steps, warmup=max(3, args.warmup), ms_per_step=ms,
                          higher_is_better=False, dtype="f32", data="synthetic",
                          config=dict(info, widths=list(widths)), cbm_products_ms=prod_ms,
                          other_ms=ms - prod_ms)))
    return 0


def build_task(args):
    """Creation benchmark of the reference (benchmark/parallel/cbm_creation.py:13-14, 42-51): build the
    structure for alpha in {0, 1, 2, 4, 8, 16, 32, 64}, report mean wall time of the constructor
    over ``--steps`` builds (the reference uses 5) and the compression ratio.  Host only."""
    import torch
    from cbm4gnn_b200 import graphs
    from cbm4gnn_b200.cbm import cbm_matrix
    from cbm4gnn_b200.utility import add_self_loops
    cfg = graphs.CONFIGS[args.workload]
    e = torch.from_numpy(graphs.make_graph(args.workload, scale=args.scale))
    if cfg["normalized"]:
        e = add_self_loops(e)
    e32, ones = e.to(torch.int32), torch.ones(e.shape[1])
    iters = max(1, min(args.steps, 5))
    rows = []
    for alpha in (0, 1, 2, 4, 8, 16, 32, 64):
        ts = []
        for _ in range(iters):
            t0 = time.perf_counter()
            c = cbm_matrix(e32, ones, alpha=alpha, normalized=cfg["normalized"])
            ts.append(time.perf_counter() - t0)
        rows.append(dict(alpha=alpha, seconds_mean=float(np.mean(ts)), seconds_std=float(np.std(ts)),
                         native_seconds=c.build_info["seconds_total"], n_delta=c.build_info["n_delta"],
                         n_candidates=c.build_info["n_candidates"], depth=c.build_info["depth"],
                         n_root_children=c.build_info["n_root_children"],
                         compression_ratio=c.compression_ratio()))
    print(json.dumps(dict(metric="cbm_creation_seconds", unit="s", higher_is_better=False, data="synthetic",
                          config=dict(workload=args.workload, n=c.num_rows, nnz=int(e.shape[1]),
                                      normalized=cfg["normalized"], host_threads=os.cpu_count(), builds_per_alpha=iters),
                          value=rows[0]["seconds_mean"], per_alpha=rows)))
    return 0


def csr_task(args):
    """The comparison the reference makes (benchmark/parallel/benchmark_spmm_cpu.py:112-150): the same
    matrix stored as plain CSR (weights deg^-1/2[row] deg^-1/2[col] when normalized) multiplied by the
    library's CSR kernel, next to the CBM product of the same workload."""
    import ctypes
    import torch
    from cbm4gnn_b200 import _lib
    from cbm4gnn_b200.alpha_search import product_bytes
    c, x, info = make_workload(args, 1)
    L = _lib.lib()
    dev = torch.device("cuda", 0)
    n, f = c.num_rows, info["f"]
    order = np.lexsort((c._col, c._row))
    row, col = c._row[order], c._col[order]
    crow = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(np.bincount(row, minlength=n), out=crow[1:])
    if c.col_multiplier is not None:
        s_ = c.col_multiplier.numpy()
        val = (s_[row] * s_[col]).astype(np.float32)
    else:
        val = np.ones(row.shape[0], dtype=np.float32)
    crow_d, col_d, val_d = (torch.from_numpy(a).to(dev) for a in (crow, col.astype(np.int32), val))
    rb, re_ = crow_d[:-1].contiguous(), crow_d[1:].contiguous()
    xd = torch.from_numpy(x).to(dev)
    y_csr, y_cbm = torch.empty((n, f), device=dev), torch.empty((n, f), device=dev)
    st = torch.cuda.current_stream().cuda_stream
    plan = c.plan(0)
    cbm_fn = L.cbm_b200_fused_spmm_update if c.normalized else L.cbm_b200_spmm_update

    def run_csr():
        _lib.check(L.cbm_b200_csr_spmm(n, rb.data_ptr(), re_.data_ptr(), col_d.data_ptr(), val_d.data_ptr(),
                                       xd.data_ptr(), f, y_csr.data_ptr(), f, f, ctypes.c_void_p(st)))

    def run_cbm():
        _lib.check(cbm_fn(plan.handle, xd.data_ptr(), f, y_cbm.data_ptr(), f, f, ctypes.c_void_p(st)))

    a_sp = torch.sparse_csr_tensor(crow_d.long(), col_d.long(), val_d, size=(n, n), check_invariants=False)

    def run_lib():  # cuSPARSE through torch, for context
        return a_sp @ xd

    out = {}
    for name, fn in (("csr", run_csr), ("cbm", run_cbm), ("cusparse", run_lib)):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / args.steps
    err = float((y_csr - y_cbm).abs().max() / max(1e-30, float(y_csr.abs().max())))
    nnz = int(row.shape[0])
    print(json.dumps(dict(metric="csr_vs_cbm_spmm_ms", unit="ms", value=out["cbm"], higher_is_better=False,
                          n_gpus=1, steps=args.steps, warmup=max(3, args.warmup), dtype="f32", data="synthetic",
                          config=info, csr_ms=out["csr"], cbm_ms=out["cbm"], cusparse_csr_ms=out["cusparse"],
                          speedup_over_csr=out["csr"] / out["cbm"], speedup_over_cusparse=out["cusparse"] / out["cbm"],
                          csr_GBps=product_bytes(n, nnz, n, f) / out["csr"] / 1e6,
                          cbm_GBps=product_bytes(n, info["n_delta"], info["n_root_children"], f) / out["cbm"] / 1e6,
                          max_rel_difference=err)))
    return 0 if err < 1e-4 else 1


def sharded_gcn_task(args, widths):
    """Forward pass of the workload's GCN stack with the structure sharded over the ranks
    (one NCCL all-gather per layer); strong scaling: the graph does not grow with N."""
    import torch
    import torch.distributed as dist
    from cbm4gnn_b200.sharding import ShardedCBM, ShardedGCN
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    args.scaling = "strong"
    c, x, info = make_workload(args, 1)
    sh = ShardedCBM(c, rank, world, device_index=local_rank)
    torch.manual_seed(0)
    model = ShardedGCN(widths, sh).to(dev)
    xl = sh.to_labels(torch.from_numpy(x).to(dev))
    for _ in range(max(3, args.warmup)):
        model(xl, gather_output=False)
    sh.plan.status()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        model(xl, gather_output=False)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    # per-layer local products alone
    per_layer = []
    for f in widths[1:]:
        a = torch.randn((sh.part.n_labels, f), device=dev)
        out = torch.zeros_like(a)
        for _ in range(3):
            sh.local_product(a, out)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(10):
            sh.local_product(a, out)
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / 10
        ab = algorithmic_bytes(sh.plan.n_rows, sh.plan.n_delta, sh.plan.n_root_children, f)
        per_layer.append(dict(f=f, ms=t, GBps=ab / t / 1e6))
    stats = torch.tensor([ms] + [d["ms"] for d in per_layer], dtype=torch.float64, device=dev)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    if rank == 0:
        for d, t in zip(per_layer, stats[1:].tolist()):
            d["ms_max_over_ranks"] = t
        print(json.dumps(dict(metric="gcn_%dlayer_fwd_ms" % (len(widths) - 1), value=stats[0].item(), unit="ms",
                              n_gpus=world, steps=args.steps, warmup=max(3, args.warmup), ms_per_step=stats[0].item(),
                              higher_is_better=False, scaling="strong", dtype="f32", data="synthetic",
                              config=dict(info, widths=list(widths), parallelism=f"subtree-sharded x{world}, "
                                          "one all-gather per layer", shard_rows=sh.part.shard_rows,
                                          rows_per_gpu=[int(v) for v in sh.part.counts]),
                              per_layer_local_product=per_layer)))
    dist.destroy_process_group()
    return 0


def main():
    args = parse()
    if args.task == "gcn":
        return gcn_task(args)
    if args.task == "build":
        return build_task(args)
    if args.task == "csr":
        return csr_task(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != max(1, args.gpus) and world > 1:
        args.gpus = world

    if args.impl == "reference":
        if rank != 0:
            return 0
        c, x, info = make_workload(args, max(1, args.gpus))
        ab = algorithmic_bytes(c.num_rows, info["n_delta"], info["n_root_children"], info["f"])
        per, iters, threads = cpu_reference(c, x, 0.0, steps=args.steps, warmup=max(1, args.warmup))
        val = ab / per / 1e9
        line = dict(impl="reference", metric="cbm_spmm_algorithmic_GBps", value=val, unit="GB/s", n_gpus=args.gpus,
                    steps=iters, warmup=max(1, args.warmup), ms_per_step=per * 1e3, higher_is_better=True,
                    scaling=args.scaling,
                    vs_baseline=None, dtype="f32", data="synthetic",
                    config=dict(info, l2="host run"),
                    cpu_baseline=dict(value=val, unit="GB/s", cores=threads, kind="port",
                                      sample=f"{iters} full products (torch CSR deltas@x + OpenMP tree update)"),
                    e2e=dict(value=val, unit="GB/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from cbm4gnn_b200 import _lib
    _lib.lib()
    c, x, info = make_workload(args, world)
    f = info["f"]
    if world > 1:
        from cbm4gnn_b200.sharding import ShardedCBM
        sh = ShardedCBM(c, rank, world, device_index=local_rank)
        plan = sh.plan
        xp = np.zeros((sh.part.n_labels, f), dtype=np.float32)
        xp[sh.part.perm] = x
        x_host = torch.from_numpy(xp).pin_memory()
        n_out = sh.part.shard_rows
    else:
        plan = c.plan(local_rank)
        x_host = torch.from_numpy(x).pin_memory()
        n_out = c.num_rows
    plan.tune(args.slab, args.blocks, args.host_chunk, args.form)
    xd = x_host.to(dev, non_blocking=True)
    yd = torch.zeros((n_out, f), device=dev)
    y_host = torch.empty((n_out, f)).pin_memory()
    fn = _lib.lib().cbm_b200_fused_spmm_update if c.normalized else _lib.lib().cbm_b200_spmm_update
    stream = torch.cuda.current_stream()

    def step():
        _lib.check(fn(plan.handle, xd.data_ptr(), f, yd.data_ptr(), f, f, stream.cuda_stream))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # nvidia-smi samples every 20 ms from before the warm-up to the end of the timed region; with
    # the default K the timed region lasts a few tens of milliseconds, so only a few samples fall
    # under load (those with GPU utilisation reported > 0 are the ones summarised)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.05)
    for _ in range(max(3, args.warmup)):
        step()
    plan.status(stream.cuda_stream)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    per_launch = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop() if rank == 0 else None
    plan.status(stream.cuda_stream)

    ab_local = algorithmic_bytes(plan.n_rows, plan.n_delta, plan.n_root_children, f)

    # end to end through the public API with host tensors: H2D of X, product, D2H of Y every step
    e2e_ms = None
    if not args.no_e2e:
        api = (lambda: c.omp_mkl_csr_fused_spmm_update(x_host, y_host)) if c.normalized else \
              (lambda: c.omp_mkl_csr_spmm_update(x_host, y_host))
        if world > 1:
            host_fn = _lib.lib().cbm_b200_spmm_update_host
            api = lambda: _lib.check(host_fn(plan.handle, x_host.data_ptr(), y_host.data_ptr(), f,
                                             1 if c.normalized else 0))
        k_e2e = max(3, min(args.steps, 10))
        api()
        barrier()
        t0 = time.perf_counter()
        for _ in range(k_e2e):
            api()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / k_e2e
        yd2 = torch.empty_like(yd)
        _lib.check(fn(plan.handle, xd.data_ptr(), f, yd2.data_ptr(), f, f, stream.cuda_stream))
        torch.cuda.synchronize()
        if not torch.equal(yd2.cpu(), y_host):
            raise SystemExit("end-to-end result differs from the device-resident result")

    stats = torch.tensor([total_ms, float(ab_local), e2e_ms or 0.0, float(np.median(per_launch))],
                         dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms_max, launch_ms = mx[0].item(), mx[2].item(), mx[3].item()
        ab_total = sm[1].item()
    else:
        e2e_ms_max, launch_ms, ab_total = (e2e_ms or 0.0), stats[3].item(), float(ab_local)

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
        ms_per_step = total_ms / args.steps
        value = ab_total / (ms_per_step * 1e-3) / 1e9
        achieved = ab_local / (launch_ms * 1e-3) / 1e9
        line = dict(metric="cbm_spmm_algorithmic_GBps", value=value, unit="GB/s", n_gpus=world, steps=args.steps,
                    warmup=max(3, args.warmup), ms_per_step=ms_per_step, higher_is_better=True, scaling=args.scaling,
                    vs_baseline=None, dtype="f32", data="synthetic",
                    config=dict(info, l2="operands (X + Y = %.0f MB) exceed the 126 MB L2; no flush" %
                                ((xd.numel() + yd.numel()) * 4 / 1e6),
                                parallelism=f"subtree-sharded x{world}" if world > 1 else "single GPU",
                                rows_per_gpu=plan.n_rows, delta_entries_per_gpu=plan.n_delta),
                    gpu_launches=args.steps,
                    roofline=dict(bound="hbm", achieved=achieved, peak=peak, unit="GB/s", frac=achieved / peak,
                                  peak_source=peak_src, traffic=None, kernel="cbm_items_kernel",
                                  algorithmic_bytes_per_launch=ab_local, launch_ms=launch_ms),
                    clocks=clocks)
        if e2e_ms is not None:
            h2d = x_host.numel() * 4
            d2h = y_host.numel() * 4
            line["e2e"] = dict(value=ab_total / (e2e_ms_max * 1e-3) / 1e9, unit="GB/s", ms_per_step=e2e_ms_max,
                               h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h)
        if world == 1 and not args.no_cpu:
            per, iters, threads = cpu_reference(c, x, args.cpu_seconds)
            line["cpu_baseline"] = dict(value=ab_total / per / 1e9, unit="GB/s", ms_per_step=per * 1e3, cores=threads,
                                        kind="port",
                                        sample=f"{iters} full products of the same workload "
                                               f"(torch CSR deltas@x + OpenMP tree update)")
        traffic = DRAM_TRAFFIC.get((info["workload"], f, world, args.scale))
        line["roofline"]["traffic"] = traffic
        if traffic:
            # the gathers are mostly served by L2, so the algorithmic rate can exceed the HBM peak;
            # the DRAM-side view of the same launch is reported next to it
            line["roofline"]["dram_achieved"] = traffic / (launch_ms * 1e-3) / 1e9
            line["roofline"]["dram_frac"] = line["roofline"]["dram_achieved"] / peak
            line["roofline"]["note"] = ("achieved = algorithmic bytes / time; X slabs are L2-resident, DRAM moved "
                                        "traffic bytes per launch (ncu), dram_frac = traffic / time / peak")
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
