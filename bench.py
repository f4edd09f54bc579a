#!/usr/bin/env python
"""Benchmark of the CBM product on B200: one step = one normalized product
``Y = D^-1/2 (A+I) D^-1/2 X`` over the whole synthetic operand.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2]

Workload (N = 1): copy-model graph, 100 000 nodes, p_copy = 0.7, 5 random links, degree cap 5 000,
self loops added, alpha = 8, X = 100 000 x 500 fp32 N(0,1) — synthetic stand-in with the shape of
the second benchmark configuration.  With N > 1 the graph has N x 100 000 nodes (same generator:
weak scaling), its root subtrees are partitioned over the ranks, every rank holds all of X and
computes its shard; the product itself needs no exchange.  Rank 0 generates the graph and builds
the structure once; the other ranks load it.

``value`` is the algorithmic byte rate of the product (delta row pointers + delta indices + one
gathered operand row per delta entry + one parent row per non-root row + Y written once + per-row
parent/scale words, divided by time).  Most of those bytes are operand rows gathered again and
again out of L2, so this rate is NOT an HBM rate; the ``roofline`` object therefore reports the
bytes that can only come from HBM (X once, Y once, indices) against the measured copy peak, the
DRAM traffic an ``ncu`` capture of the same kernel build counted, and the gather rate against the
L2-to-SM bandwidth measured live by a streaming read of an L2-resident buffer.

The same JSON line carries: ``parity`` (sampled output rows against a float64 CSR product; the run
fails above the tolerance), ``e2e`` (host tensors through the public API, copies inside the timed
region), ``cpu_baseline`` / ``cpu_baseline_sequential`` (the reference's own OpenMP + oneMKL path and
its sequential path on the host cores), ``sustained`` (a loop of at least half a second with the
clocks sampled over it) and ``extras``: at N = 1 the 2-layer GCN forward + backward of the third
configuration and the product of the fourth; at N > 1 strong-scaling records of the fourth
configuration's product and the fifth configuration's 3-layer forward.

``--impl reference`` times the reference's own CPU path for the same product on the host cores:
the unmodified native module compiled into oracle/_ref when present (kind "reference"), else the
restatement (kind "port": torch CSR ``deltas @ x`` = oneMKL inside libtorch + restated tree update).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "cbm_spmm_algorithmic_GBps"
TOL_ATOL = TOL_RTOL = 1e-4  # tests/test_matmul_correctness.py:43 of the reference


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
    ap.add_argument("--no-extras", action="store_true", help="skip the sub-records of the other configurations")
    ap.add_argument("--contiguous", action="store_true",
                    help="device-resident X and Y with a row pitch of exactly F floats instead of whole 128-byte lines")
    ap.add_argument("--build-gpu", action="store_true", help="--task build: candidate search on the GPU")
    ap.add_argument("--bare", action="store_true",
                    help="warm-up and timed launches only (no parity sample, sustained loop, L2 probe, end-to-end, "
                         "CPU baselines or sub-records): the command line profiler captures run")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    return ap.parse_args()


def algorithmic_bytes(n_rows, n_delta, n_root_children, f):
    """Bytes one product must move: 4(N+1) row pointers + 4 nnzD indices + 4 F nnzD gathered rows
    + 4 F (N - roots) parent rows + 4 F N output + 8 N parent/scale words."""
    from cbm4gnn_b200.alpha_search import product_bytes
    return product_bytes(n_rows, n_delta, n_root_children, f)


def compulsory_bytes(n_rows, n_labels, n_delta, f):
    """Bytes that have to cross the HBM interface at least once: X once, Y once, one index word per
    delta entry, 12 bytes of per-row words."""
    return 4 * f * n_labels + 4 * f * n_rows + 4 * n_delta + 12 * n_rows


def engine_fingerprint() -> str:
    """git blob hash of the kernel source: ties an ncu byte count to the build it was taken on."""
    data = open(os.path.join(ROOT, "cbm4gnn_b200", "csrc", "cbm_engine.cu"), "rb").read()
    return hashlib.sha1(b"blob %d\0" % len(data) + data).hexdigest()


def recorded_traffic(workload, f, n_gpus, scale, alpha):
    """DRAM bytes per launch of the product kernel from the tracked ncu summaries
    (profiles/dram_traffic.json), only when the capture was made on this build of the kernel."""
    try:
        table = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))
    except Exception:
        return None, "no tracked capture"
    fp = engine_fingerprint()
    for e in table.get("captures", []):
        if (e["workload"], e["f"], e["n_gpus"], float(e["scale"]), e.get("alpha")) == (workload, f, n_gpus, float(scale), alpha):
            if e["engine_blob"] == fp:
                return e, None
            return None, "the tracked capture (%s) belongs to another build of the kernel" % e["engine_blob"][:10]
    return None, "no tracked capture of this workload"


# --------------------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------------------
def _rank_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def build_structure(name, scale, alpha=None, world_nodes=1, share=True, build_device=None):
    """The graph of a configuration and its CBM structure.  Under torchrun rank 0 generates and
    builds with every host core and leaves the result in shared memory; the other ranks wait for it
    (N ranks building the same structure with 1/N of the cores each took N times as long)."""
    import torch
    from cbm4gnn_b200 import graphs
    from cbm4gnn_b200.cbm import cbm_matrix
    from cbm4gnn_b200.utility import add_self_loops
    rank, world, _ = _rank_env()
    cfg = dict(graphs.CONFIGS[name])
    if alpha is not None and alpha >= 0:
        cfg["alpha"] = alpha
    tag = "%s_%s_%g_%d_%d" % (os.environ.get("MASTER_PORT", "solo"), name, scale, cfg["alpha"], world_nodes)
    shm = "/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir()
    path = os.path.join(shm, "cbm_bench_%s.pt" % tag)
    times = dict(graph_seconds=None, build_seconds=None)
    if rank == 0 or not share or world == 1:
        t0 = time.time()
        if cfg["kind"] == "copy":
            n = max(64, int(cfg["n"] * scale)) * world_nodes
            ei = graphs.copy_model(n, cfg["p_copy"], cfg["n_random"], cfg["seed"], cfg["max_degree"])
        else:
            ei = graphs.make_graph(name, scale=scale * world_nodes)
        e = torch.from_numpy(ei)
        if cfg["normalized"]:
            e = add_self_loops(e)
        t1 = time.time()
        c = cbm_matrix(e.to(torch.int32), torch.ones(e.shape[1]), alpha=cfg["alpha"], normalized=cfg["normalized"],
                       n_threads=os.cpu_count() or 1, build_device=build_device)
        times = dict(graph_seconds=round(t1 - t0, 2), build_seconds=round(c.build_info["seconds_total"], 3),
                     candidates_on_gpu=c.build_info.get("candidates_on_gpu", False),
                     candidates_seconds=round(c.build_info["seconds_candidates"], 3),
                     arborescence_seconds=round(c.build_info["seconds_arborescence"], 3),
                     builder_threads=os.cpu_count() or 1)
        if world > 1 and share:
            c.save(path + ".tmp")
            os.replace(path + ".tmp", path)
    else:
        deadline = time.time() + 3600
        while not os.path.exists(path):
            if time.time() > deadline:
                raise SystemExit("rank %d: the structure never arrived from rank 0" % rank)
            time.sleep(0.25)
        c = cbm_matrix.load(path)
    return c, cfg, times, path


def workload_config(name, c, cfg, f):
    """The keys that define the workload — identical in both arms of the benchmark."""
    return dict(workload=name, n=c.num_rows, nnz=c.nnz, f=f, alpha=cfg["alpha"], normalized=cfg["normalized"],
                n_delta=c.build_info["n_delta"], n_root_children=c.build_info["n_root_children"],
                depth=c.build_info["depth"],
                l2=("operands (X + Y = %.0f MB) exceed the 126 MB L2; no flush" if 2 * c.num_rows * f * 4 > 126e6 else
                    "operands (X + Y = %.0f MB) fit the 126 MB L2 and are not flushed: a reduced-size run, not a bench value")
                % (2 * c.num_rows * f * 4 / 1e6))


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
        sm, util, reasons, mx, power = [], [], set(), None, []
        try:
            for line in open(self.path):
                p = [t.strip() for t in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    mx = float(p[2])
                    power.append(float(p[3]))
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
                       samples_under_load=len([u for u in util if u > 0]), power_w_max=max(power) if power else None)
        return out


# --------------------------------------------------------------------------------------------------
# the reference's CPU path
# --------------------------------------------------------------------------------------------------
def cpu_reference(c, x, seconds, threads=None, steps=None, warmup=1, sequential=False):
    """The reference's CPU product on the host cores; returns (seconds per product, products timed,
    threads, kind).  With oracle/_ref present this is the reference's unmodified compiled code
    (omp_/seq_s_*spmm_update_csr_int32: oneMKL product + its own tree update, kind "reference");
    otherwise the restatement (kind "port").  Either exactly ``steps`` products after ``warmup``,
    or (steps None) repeated for about ``seconds``."""
    import torch
    from oracle import cbm_oracle as orc
    from oracle import reference
    threads = 1 if sequential else (threads or os.cpu_count())
    torch.set_num_threads(threads)
    orc.clib().oracle_set_threads(threads)
    xt = torch.from_numpy(x)
    mult = None if c.col_multiplier is None else c.col_multiplier
    if reference.ref_available():
        ref = reference.ref_module()
        crow = torch.from_numpy(c._crow)
        rb, re_ = crow[:-1].contiguous(), crow[1:].contiguous()
        col, val = torch.from_numpy(c._dcol), torch.from_numpy(c._dval)
        y = torch.zeros_like(xt)
        pre = "seq" if sequential else "omp"
        kind = "reference"
        if mult is None:
            fn = getattr(ref, pre + "_s_spmm_update_csr_int32")
            once = lambda: fn(rb, re_, col, val, xt, c.mst_row, c.mst_col, y)
        else:
            fn = getattr(ref, pre + "_s_fused_spmm_update_csr_int32")
            once = lambda: fn(rb, re_, col, val, xt, c.mst_row, c.mst_col, mult, y)
    else:
        kind = "port"
        mr, mc = c.mst_row.numpy(), c.mst_col.numpy()

        def once():
            y = (c.deltas @ xt).numpy()
            if mult is None:
                orc.update(mr, mc, y, parallel=not sequential)
            else:
                orc.fused_update(mr, mc, mult.numpy(), y, parallel=not sequential)

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
    torch.set_num_threads(os.cpu_count() or 1)
    return el / it, it, threads, kind


def sample_parity(ei_row, ei_col, n, mult, x, rows, got_rows):
    """Sampled rows of the product against float64 CSR.  Returns the record for the JSON line;
    ``max_err_over_tol`` <= 1 means every element is within atol + rtol |want|."""
    import scipy.sparse as sp
    a = sp.csr_matrix((np.ones(ei_row.shape[0], dtype=np.float64), (ei_row, ei_col)), shape=(n, n))
    sub = a[rows]
    if mult is not None:
        s = mult.astype(np.float64)
        sub = sp.diags(s[rows]) @ sub @ sp.diags(s)
    want = np.asarray(sub @ x.astype(np.float64))
    d = np.abs(got_rows.astype(np.float64) - want)
    return dict(rows=int(len(rows)), against="float64 csr", max_abs_err=float(d.max()),
                max_rel_err=float(d.max() / max(1e-30, np.abs(want).max())),
                max_err_over_tol=float((d / (TOL_ATOL + TOL_RTOL * np.abs(want))).max()), atol=TOL_ATOL, rtol=TOL_RTOL)


# --------------------------------------------------------------------------------------------------
# tasks other than the headline
# --------------------------------------------------------------------------------------------------
def gcn_fwd_bwd(c, cfg, x, steps, warmup, dev):
    """Forward + backward of the configuration's GCN stack (ReLU between layers, loss = sum of
    outputs; protocol of benchmark/parallel/benchmark_gcn_cpu.py:92-103) and the share of it spent
    in CBM products."""
    import torch
    from cbm4gnn_b200 import _lib
    from cbm4gnn_b200.gcn import GCNModel
    widths = cfg.get("widths", (cfg["f"], 256, 64))
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

    for _ in range(max(3, warmup)):
        step()
    c.plan(dev.index).status()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    ms_weights_only = None
    if train:
        # the usual training case: the input features need no gradient, so the backward pass of the
        # first layer stops at its weight gradient (no input-gradient map, no transposed product)
        xd.requires_grad_(False)
        for _ in range(3):
            step()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms_weights_only = e0.elapsed_time(e1) / steps
        xd.requires_grad_(True)
    plan, L = c.plan(dev.index), _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    prod_ms = 0.0
    prod_widths = list(model.product_widths()) * (2 if train else 1)
    for f in prod_widths:
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
    return dict(ms=ms, train=train, widths=list(widths), product_widths=prod_widths, cbm_products_ms=prod_ms,
                other_ms=ms - prod_ms, steps=steps, ms_without_input_gradient=ms_weights_only,
                gradients="weights and input features")


def gcn_task(args):
    import torch
    from cbm4gnn_b200 import graphs
    cfg0 = graphs.CONFIGS[args.workload]
    widths = cfg0.get("widths", (cfg0["f"], 256, 64))
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return sharded_gcn_task(args, widths)
    c, cfg, times, _ = build_structure(args.workload, args.scale, args.alpha)
    x = graphs.make_features(args.workload, c.num_rows, f=widths[0])
    dev = torch.device("cuda", 0)
    r = gcn_fwd_bwd(c, cfg, x, args.steps, args.warmup, dev)
    print(json.dumps(dict(metric="gcn_%dlayer_%s_ms" % (len(widths) - 1, "fwd_bwd" if r["train"] else "fwd"),
                          value=r["ms"], unit="ms", n_gpus=1, steps=args.steps, warmup=max(3, args.warmup),
                          ms_per_step=r["ms"], higher_is_better=False, dtype="f32", data="synthetic",
                          config=dict(workload_config(args.workload, c, cfg, widths[0]), widths=list(widths)),
                          build=times, cbm_products_ms=r["cbm_products_ms"], other_ms=r["other_ms"],
                          gradients=r["gradients"], ms_without_input_gradient=r["ms_without_input_gradient"])))
    return 0


def build_task(args):
    """Creation benchmark of the reference (benchmark/parallel/cbm_creation.py:13-14, 42-51): build the
    structure for alpha in {0, 1, 2, 4, 8, 16, 32, 64}, report mean wall time of the constructor
    over ``--steps`` builds (the reference uses 5), the split between candidate search and
    arborescence, and the compression ratio.  Host only."""
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
    build_device = 0 if (args.build_gpu and torch.cuda.is_available()) else None
    alphas = (0, 1, 2, 4, 8, 16, 32, 64) if args.alpha < 0 else (args.alpha,)
    for alpha in alphas:
        ts = []
        for _ in range(iters):
            t0 = time.perf_counter()
            c = cbm_matrix(e32, ones, alpha=alpha, normalized=cfg["normalized"], build_device=build_device)
            ts.append(time.perf_counter() - t0)
        rows.append(dict(alpha=alpha, seconds_mean=float(np.mean(ts)), seconds_std=float(np.std(ts)),
                         native_seconds=c.build_info["seconds_total"],
                         candidates_on_gpu=c.build_info.get("candidates_on_gpu", False),
                         candidates_seconds=c.build_info["seconds_candidates"],
                         arborescence_seconds=c.build_info["seconds_arborescence"],
                         deltas_seconds=c.build_info["seconds_deltas"], n_delta=c.build_info["n_delta"],
                         n_candidates=c.build_info["n_candidates"], depth=c.build_info["depth"],
                         n_root_children=c.build_info["n_root_children"],
                         compression_ratio=c.compression_ratio()))
    print(json.dumps(dict(metric="cbm_creation_seconds", unit="s", higher_is_better=False, data="synthetic",
                          config=dict(workload=args.workload, n=c.num_rows, nnz=int(e.shape[1]),
                                      normalized=cfg["normalized"], host_threads=os.cpu_count(), builds_per_alpha=iters),
                          value=rows[0]["seconds_mean"], per_alpha=rows)))
    return 0


def csr_compare(c, x, steps, warmup, dev):
    """The comparison the reference makes (benchmark/parallel/benchmark_spmm_cpu.py:112-150): the same
    matrix stored as plain CSR (weights deg^-1/2[row] deg^-1/2[col] when normalized) multiplied by
    the library's CSR entry point and by cuSPARSE (through torch), next to the CBM product."""
    import ctypes
    import torch
    from cbm4gnn_b200 import _lib
    L = _lib.lib()
    n, f = c.num_rows, x.shape[1]
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
    plan = c.plan(dev.index)
    cbm_fn = L.cbm_b200_fused_spmm_update if c.normalized else L.cbm_b200_spmm_update

    from cbm4gnn_b200.cbm import csr_matrix_plan
    csr_plan = csr_matrix_plan(crow, col.astype(np.int32), val, n, dev.index)
    y_arr = torch.empty((n, f), device=dev)

    def run_csr():  # through a plan: long rows cut into segments and balanced
        csr_plan.matmul(xd, out=y_csr)

    def run_csr_arrays():  # array form, one warp per whole row
        _lib.check(L.cbm_b200_csr_spmm(n, rb.data_ptr(), re_.data_ptr(), col_d.data_ptr(), val_d.data_ptr(),
                                       xd.data_ptr(), f, y_arr.data_ptr(), f, f, ctypes.c_void_p(st)))

    def run_cbm():
        _lib.check(cbm_fn(plan.handle, xd.data_ptr(), f, y_cbm.data_ptr(), f, f, ctypes.c_void_p(st)))

    a_sp = torch.sparse_csr_tensor(crow_d.long(), col_d.long(), val_d, size=(n, n), check_invariants=False)
    out = {}
    for name, fn in (("csr", run_csr), ("csr_arrays", run_csr_arrays), ("cbm", run_cbm), ("cusparse", lambda: a_sp @ xd)):
        for _ in range(max(3, warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / steps
    err = float((y_csr - y_cbm).abs().max() / max(1e-30, float(y_csr.abs().max())))
    err = max(err, float((y_arr - y_cbm).abs().max() / max(1e-30, float(y_csr.abs().max()))))
    return dict(csr_ms=out["csr"], csr_arrays_ms=out["csr_arrays"], cbm_ms=out["cbm"], cusparse_csr_ms=out["cusparse"],
                speedup_over_cusparse=out["cusparse"] / out["cbm"], own_csr_over_cusparse=out["cusparse"] / out["csr"],
                max_rel_difference=err, nnz=int(row.shape[0]))


def csr_task(args):
    import torch
    from cbm4gnn_b200 import graphs
    c, cfg, times, _ = build_structure(args.workload, args.scale, args.alpha)
    f = args.f or cfg["f"]
    x = graphs.make_features(args.workload, c.num_rows, f=f)
    r = csr_compare(c, x, args.steps, args.warmup, torch.device("cuda", 0))
    print(json.dumps(dict(metric="csr_vs_cbm_spmm_ms", unit="ms", value=r["cbm_ms"], higher_is_better=False,
                          n_gpus=1, steps=args.steps, warmup=max(3, args.warmup), dtype="f32", data="synthetic",
                          config=workload_config(args.workload, c, cfg, f), build=times, **r)))
    return 0 if r["max_rel_difference"] < 1e-4 else 1


def sharded_gcn_forward(c, cfg, name, steps, warmup, dev, rank, world, group=None):
    """Strong-scaling record: forward pass of the configuration's GCN stack with the structure's
    root subtrees sharded over the ranks; per layer the local product, the exchange and the dense
    map, each as the maximum over ranks, and sampled rows of the result against float64 CSR."""
    import torch
    import torch.distributed as dist
    from cbm4gnn_b200 import graphs
    from cbm4gnn_b200.sharding import ShardedCBM, ShardedGCN
    widths = cfg["widths"]
    sh = ShardedCBM(c, rank, world, device_index=dev.index, group=group)
    torch.manual_seed(0)
    model = ShardedGCN(widths, sh).to(dev)
    x = graphs.make_features(name, c.num_rows, f=widths[0])
    xl = sh.to_labels(torch.from_numpy(x).to(dev))
    for _ in range(max(3, warmup)):
        model(xl, gather_output=False)
    sh.plan.status()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = model(xl, gather_output=False)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    phases = model.timed_forward(xl)  # per layer: product / exchange / dense map, device-timed
    # parity of this rank's rows: the whole stack in float64 on sampled rows is costly, so the
    # last layer's product is checked given the model's own input to it
    par = model.check_last_product(xl, rows=500)
    stats = torch.tensor([ms, par["max_err_over_tol"], par["max_rel_err"]] + [v for p in phases for v in
                                                                             (p["product_ms"], p["exchange_ms"], p["dense_ms"])],
                         dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    s = stats.tolist()
    layers = []
    for i, p in enumerate(phases):
        ab = algorithmic_bytes(sh.plan.n_rows, sh.plan.n_delta, sh.plan.n_root_children, p["product_width"])
        layers.append(dict(layer=i, order=p["order"], product_width=p["product_width"], product_ms=s[3 + 3 * i],
                           exchange_ms=s[4 + 3 * i], dense_ms=s[5 + 3 * i], exchange_width=p["exchange_width"],
                           product_GBps_rank0=ab / (p["product_ms"] * 1e-3) / 1e9))
    return dict(workload=name, n=c.num_rows, n_delta=c.build_info["n_delta"], widths=list(widths), n_gpus=world,
                ms=s[0], steps=steps, scaling="strong", layers=layers,
                parity=dict(rows=par["rows"] * world, against="float64 csr of the last layer's product",
                            max_err_over_tol=s[1], max_rel_err=s[2]))


def sharded_gcn_task(args, widths):
    import torch
    import torch.distributed as dist
    rank, world, local_rank = _rank_env()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    c, cfg, times, path = build_structure(args.workload, args.scale, args.alpha)
    r = sharded_gcn_forward(c, cfg, args.workload, args.steps, args.warmup, dev, rank, world)
    if rank == 0:
        print(json.dumps(dict(metric="gcn_%dlayer_fwd_ms" % (len(widths) - 1), value=r["ms"], unit="ms", n_gpus=world,
                              steps=args.steps, warmup=max(3, args.warmup), ms_per_step=r["ms"],
                              higher_is_better=False, scaling="strong", dtype="f32", data="synthetic",
                              config=dict(workload_config(args.workload, c, cfg, widths[0]), widths=list(widths)),
                              build=times, layers=r["layers"], parity=r["parity"])))
    dist.barrier()
    if rank == 0 and os.path.exists(path):
        os.unlink(path)
    dist.destroy_process_group()
    return 0 if r["parity"]["max_err_over_tol"] <= 1.0 else 1


def sharded_spmm(c, cfg, name, steps, warmup, dev, rank, world):
    """Strong-scaling record of one product: the structure's root subtrees sharded over the ranks,
    every rank holding all of X; time = max over ranks, sampled owned rows against float64 CSR."""
    import torch
    import torch.distributed as dist
    from cbm4gnn_b200 import _lib, graphs
    from cbm4gnn_b200.sharding import ShardedCBM
    f = cfg["f"]
    sh = ShardedCBM(c, rank, world, device_index=dev.index)
    x = graphs.make_features(name, c.num_rows, f=f)
    xl = sh.to_labels(torch.from_numpy(x).to(dev))
    out = torch.zeros((sh.part.n_labels, f), device=dev)
    for _ in range(max(3, warmup)):
        sh.local_product(xl, out)
    sh.plan.status()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        sh.local_product(xl, out)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    par = shard_parity(c, sh, x, out, 1000 // world + 1, seed=rank)
    ab = algorithmic_bytes(sh.plan.n_rows, sh.plan.n_delta, sh.plan.n_root_children, f)
    exchange = None
    if world > 1:
        exchange = product_with_exchange(sh, xl, out, f, steps, dev)
    stats = torch.tensor([ms, par["max_err_over_tol"], par["max_rel_err"]], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(ab), float(par["rows"])], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    return dict(workload=name, n=c.num_rows, n_delta=c.build_info["n_delta"], f=f, alpha=cfg["alpha"], n_gpus=world,
                ms=stats[0].item(), steps=steps, scaling="strong", algorithmic_GBps=tot[0].item() / (stats[0].item() * 1e-3) / 1e9,
                product_plus_exchange=exchange,
                parity=dict(rows=int(tot[1].item()), against="float64 csr", max_err_over_tol=stats[1].item(),
                            max_rel_err=stats[2].item()))


def product_with_exchange(sh, xl, out, f, steps, dev):
    """The product followed by the exchange that hands its result to every GPU (what a layer output
    needs), two ways: the product, then an NCCL all-gather of the shards; and the product kernel
    delivering every finished row itself into all GPUs' gathered buffers (ordinary peer stores over
    NVLink while the product runs) followed by one barrier.  Times are the maximum over ranks."""
    import torch
    import torch.distributed as dist
    res = {}

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def nccl():
        mine = sh.local_product(xl, out)
        dist.all_gather_into_tensor(out, mine, group=sh.group)

    res["nccl_ms"] = timed(nccl)
    want = out.clone()
    try:
        from cbm4gnn_b200.sharding import PeerBuffer
        pb = PeerBuffer(sh.part.n_labels, f, dev, sh.group)
        raw = torch.zeros((sh.part.shard_rows, f), device=dev)
        dst = pb.slice_addresses(sh.begin)

        def fused():
            pb.barrier()
            sh.product_into(xl, raw, bcast=dst)
            pb.barrier()

        res["fused_peer_store_ms"] = timed(fused)
        same = torch.tensor([1.0 if torch.equal(pb.tensor, want) else 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        res["fused_equals_nccl"] = bool(same.item() == 1.0)
    except Exception as e:  # symmetric memory not available on this box: the NCCL figure stands alone
        res["fused_peer_store_ms"] = None
        res["note"] = "peer-store delivery not measured: " + str(e).splitlines()[0][:200]
    return res


def shard_parity(c, sh, x, out_labels, n_rows, seed=0):
    """Sampled rows this rank owns (device result in label space) against float64 CSR."""
    lab = sh.part.perm
    own = np.nonzero((lab >= sh.begin) & (lab < sh.end))[0]
    rows = np.sort(np.random.default_rng(1234 + seed).choice(own, min(n_rows, own.size), replace=False))
    import torch
    got = out_labels[torch.from_numpy(lab[rows].astype(np.int64)).to(out_labels.device)].cpu().numpy()
    mult = None if c.col_multiplier is None else c.col_multiplier.numpy()
    return sample_parity(c._row, c._col, c.num_rows, mult, x, rows, got)


# --------------------------------------------------------------------------------------------------
# the headline
# --------------------------------------------------------------------------------------------------
def main():
    args = parse()
    if args.task == "gcn":
        return gcn_task(args)
    if args.task == "build":
        return build_task(args)
    if args.task == "csr":
        return csr_task(args)
    rank, world, local_rank = _rank_env()
    if world != max(1, args.gpus) and world > 1:
        args.gpus = world
    if args.bare:
        args.no_e2e = args.no_cpu = args.no_extras = True
    from cbm4gnn_b200 import graphs

    if args.impl == "reference":
        if rank != 0:
            return 0
        nodes = 1 if args.scaling == "strong" else max(1, args.gpus)
        c, cfg, times, _ = build_structure(args.workload, args.scale, args.alpha, world_nodes=nodes, share=False)
        f = args.f or cfg["f"]
        x = graphs.make_features(args.workload, c.num_rows, f=f)
        ab = algorithmic_bytes(c.num_rows, c.build_info["n_delta"], c.build_info["n_root_children"], f)
        per, iters, threads, kind = cpu_reference(c, x, 0.0, steps=args.steps, warmup=max(1, args.warmup))
        val = ab / per / 1e9
        what = ("the reference's compiled omp_s_%sspmm_update_csr_int32 (oneMKL product + OpenMP tree update)" %
                ("fused_" if c.normalized else "")) if kind == "reference" else "torch CSR deltas@x + restated OpenMP tree update"
        line = dict(impl="reference", metric=METRIC, value=val, unit="GB/s", n_gpus=args.gpus,
                    steps=iters, warmup=max(1, args.warmup), ms_per_step=per * 1e3, higher_is_better=True,
                    scaling=args.scaling, vs_baseline=None, dtype="f32", data="synthetic",
                    config=workload_config(args.workload, c, cfg, f), build=times,
                    cpu_baseline=dict(value=val, unit="GB/s", cores=threads, kind=kind,
                                      sample=f"{iters} full products: {what}"),
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
    L = _lib.lib()
    nodes = 1 if args.scaling == "strong" else world
    c, cfg, times, shared_path = build_structure(args.workload, args.scale, args.alpha, world_nodes=nodes,
                                                 build_device=local_rank)
    f = args.f or cfg["f"]
    x = graphs.make_features(args.workload, c.num_rows, f=f)
    sh = None
    if world > 1:
        from cbm4gnn_b200.sharding import ShardedCBM
        sh = ShardedCBM(c, rank, world, device_index=local_rank)
        plan = sh.plan
        xp = np.zeros((sh.part.n_labels, f), dtype=np.float32)
        xp[sh.part.perm] = x
        x_host = torch.from_numpy(xp).pin_memory()
        n_out, n_labels = sh.part.shard_rows, sh.part.n_labels
    else:
        plan = c.plan(local_rank)
        x_host = torch.from_numpy(x).pin_memory()
        n_out = n_labels = c.num_rows
    plan.tune(args.slab, args.blocks, args.host_chunk, args.form)
    # device-resident operand and result in the library's recommended layout: rows pitched to whole
    # 128-byte lines (cbm4gnn_b200.cbm.aligned_rows); --contiguous keeps the pitch at F floats
    from cbm4gnn_b200.cbm import aligned_rows
    if args.contiguous:
        xd = x_host.to(dev, non_blocking=True)
        yd = torch.zeros((n_out, f), device=dev)
    else:
        xd = aligned_rows(x_host.size(0), f, dev)
        xd.copy_(x_host, non_blocking=True)
        yd = aligned_rows(n_out, f, dev)
    ldx, ldy = xd.stride(0), yd.stride(0)
    y_host = torch.empty((n_out, f)).pin_memory()
    fn = L.cbm_b200_fused_spmm_update if c.normalized else L.cbm_b200_spmm_update
    stream = torch.cuda.current_stream()

    def step():
        _lib.check(fn(plan.handle, xd.data_ptr(), ldx, yd.data_ptr(), ldy, f, stream.cuda_stream))

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

    # parity of what was just timed: sampled owned rows against float64 CSR
    if args.bare:
        parity = dict(rows=0, max_err_over_tol=0.0, max_rel_err=0.0, max_abs_err=0.0)
    elif sh is not None:
        full = torch.zeros((n_labels, f), device=dev)
        full[sh.begin:sh.end] = yd
        parity = shard_parity(c, sh, x, full, 1000 // world + 1, seed=rank)
        del full
    else:
        rows = np.sort(np.random.default_rng(1234).choice(c.num_rows, min(1000, c.num_rows), replace=False))
        mult = None if c.col_multiplier is None else c.col_multiplier.numpy()
        parity = sample_parity(c._row, c._col, c.num_rows, mult, x, rows,
                               yd[torch.from_numpy(rows).to(dev)].cpu().numpy())

    ab_local = algorithmic_bytes(plan.n_rows, plan.n_delta, plan.n_root_children, f)

    # sustained: back-to-back products for at least half a second, clocks sampled over the loop
    sustained = None
    if world == 1 and not args.bare:
        n_loop = max(args.steps, int(0.6 / max(1e-6, total_ms / args.steps * 1e-3)) + 1)
        s2 = ClockSampler(local_rank)
        s2.start()
        time.sleep(0.05)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_loop):
            step()
        e1.record()
        torch.cuda.synchronize()
        ck = s2.stop()
        sustained = dict(ms_per_step=e0.elapsed_time(e1) / n_loop, steps=n_loop, sm_mhz=ck.get("sm_mhz"),
                         reasons=ck.get("reasons"), power_w_max=ck.get("power_w_max"))

    # end to end through the public API with host tensors: H2D of X, product, D2H of Y every step.
    # N = 1: cbm_matrix.omp_mkl_csr_fused_spmm_update(x_cpu, y_cpu).  N > 1: ShardedCBM.host_product —
    # every rank sends only its own block of X over PCIe, an all-gather over NVLink completes the
    # operand on every GPU, then the product and the D2H of the rank's own rows.
    e2e_ms = None
    h2d = d2h = 0
    if not args.no_e2e:
        if world > 1:
            x_mine = x_host[sh.begin:sh.end]
            api = lambda: sh.host_product(x_mine, y_host)
            h2d, d2h = x_mine.numel() * 4, y_host.numel() * 4
        else:
            api = (lambda: c.omp_mkl_csr_fused_spmm_update(x_host, y_host)) if c.normalized else \
                  (lambda: c.omp_mkl_csr_spmm_update(x_host, y_host))
            h2d, d2h = x_host.numel() * 4, y_host.numel() * 4
        k_e2e = max(3, min(args.steps, 10))
        api()
        barrier()
        t0 = time.perf_counter()
        for _ in range(k_e2e):
            api()
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / k_e2e
        if not torch.equal(yd.cpu(), y_host):
            raise SystemExit("end-to-end result differs from the device-resident result")

    stats = torch.tensor([total_ms, e2e_ms or 0.0, float(np.median(per_launch)), parity["max_err_over_tol"],
                          parity["max_rel_err"], parity["max_abs_err"]], dtype=torch.float64, device=dev)
    sums = torch.tensor([float(ab_local), float(parity["rows"]), float(h2d), float(d2h)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms_max, launch_ms = stats[0].item(), stats[1].item(), stats[2].item()
    ab_total = sums[0].item()
    parity = dict(rows=int(sums[1].item()), against="float64 csr", max_err_over_tol=stats[3].item(),
                  max_rel_err=stats[4].item(), max_abs_err=stats[5].item(), atol=TOL_ATOL, rtol=TOL_RTOL)

    line = None
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
        comp = compulsory_bytes(plan.n_rows, n_labels, plan.n_delta, f)
        comp_rate = comp / (launch_ms * 1e-3) / 1e9
        gather_bytes = 4 * f * plan.n_delta
        l2_rate = 0.0 if args.bare else L.cbm_b200_probe_l2_read_gbps(local_rank)
        roof = dict(bound="hbm", achieved=comp_rate, peak=peak, unit="GB/s", frac=comp_rate / peak, peak_source=peak_src,
                    kernel="cbm_items_kernel", launch_ms=launch_ms, compulsory_bytes_per_launch=comp,
                    what="achieved = bytes that must cross HBM at least once (X once + Y once + indices) / launch time",
                    algorithmic_bytes_per_launch=ab_local, l2_served_rate=ab_local / (launch_ms * 1e-3) / 1e9,
                    gather=dict(bytes_per_launch=gather_bytes, rate=gather_bytes / (launch_ms * 1e-3) / 1e9,
                                l2_to_sm_peak=l2_rate, frac=(gather_bytes / (launch_ms * 1e-3) / 1e9) / l2_rate if l2_rate > 0 else None,
                                unit="GB/s", what="operand rows gathered per launch against the rate at which all SMs "
                                                  "stream an L2-resident buffer (measured in this run)"))
        # which resource actually bounds the kernel, said in so many words for the reader of the line
        roof["binding_resource"] = "l2_to_sm (operand rows are gathered out of L2; HBM carries only the compulsory bytes)"
        roof["frac_of_binding_resource"] = roof["gather"]["frac"]
        cap, why = recorded_traffic(args.workload, f, world, args.scale, cfg["alpha"])
        if cap is not None:
            roof["traffic"] = cap["dram_bytes_per_launch"]
            roof["dram_achieved"] = cap["dram_bytes_per_launch"] / (launch_ms * 1e-3) / 1e9
            roof["dram_frac"] = roof["dram_achieved"] / peak
            roof["traffic_source"] = dict(file="profiles/dram_traffic.json", summary=cap.get("summary"),
                                          engine_blob=cap["engine_blob"])
        else:
            roof["traffic"] = None
            roof["traffic_note"] = why
        line = dict(metric=METRIC, value=value, unit="GB/s", n_gpus=world, steps=args.steps,
                    warmup=max(3, args.warmup), ms_per_step=ms_per_step, higher_is_better=True, scaling=args.scaling,
                    vs_baseline=None, dtype="f32", data="synthetic",
                    config=workload_config(args.workload, c, cfg, f),
                    parallelism=f"root subtrees sharded over {world} GPUs, X replicated" if world > 1 else "single GPU",
                    rows_per_gpu=plan.n_rows, delta_entries_per_gpu=plan.n_delta, build=times,
                    device_layout="row pitch %d floats (%s)" % (ldx, "contiguous" if ldx == f else "whole 128-byte lines"),
                    gpu_launches=args.steps, roofline=roof, parity=parity, clocks=clocks, sustained=sustained)
        if e2e_ms is not None:
            line["e2e"] = dict(value=ab_total / (e2e_ms_max * 1e-3) / 1e9, unit="GB/s", ms_per_step=e2e_ms_max,
                               h2d_bytes_per_step=int(sums[2].item()), d2h_bytes_per_step=int(sums[3].item()),
                               path="cbm_matrix.omp_mkl_csr_fused_spmm_update(x_cpu, y_cpu)" if world == 1 else
                                    "ShardedCBM.host_product, per 128-column chunk: own block H2D, NCCL all-gather, "
                                    "product, D2H, chunks pipelined")
        if world == 1 and not args.no_cpu:
            per, iters, threads, kind = cpu_reference(c, x, args.cpu_seconds)
            line["cpu_baseline"] = dict(value=ab_total / per / 1e9, unit="GB/s", ms_per_step=per * 1e3, cores=threads,
                                        kind=kind, sample=f"{iters} full products of the same workload, OpenMP + oneMKL path")
            per1, it1, _, kind1 = cpu_reference(c, x, args.cpu_seconds / 2, sequential=True)
            line["cpu_baseline_sequential"] = dict(value=ab_total / per1 / 1e9, unit="GB/s", ms_per_step=per1 * 1e3,
                                                   cores=1, kind=kind1,
                                                   sample=f"{it1} full products of the same workload, sequential path")
    del xd, yd, x_host, y_host

    # sub-records of the other configurations (same process, after the headline's timed regions)
    extras = {}
    if not args.no_extras and args.scale == 1.0 and args.workload == "c2":
        if world == 1:
            c3, cfg3, t3, _ = build_structure("c3", 1.0, build_device=local_rank)
            x3 = graphs.make_features("c3", c3.num_rows, f=cfg3["widths"][0])
            g = gcn_fwd_bwd(c3, cfg3, x3, 10, 3, dev)
            extras["gcn_c3_fwd_bwd_ms"] = g["ms"]
            extras["gcn_c3"] = dict(g, n=c3.num_rows, n_delta=c3.build_info["n_delta"], build=t3)
            del c3, x3
            c4, cfg4, t4, _ = build_structure("c4", 1.0, build_device=local_rank)
            r4 = sharded_spmm(c4, cfg4, "c4", 20, 5, dev, 0, 1)
            x4 = graphs.make_features("c4", c4.num_rows, f=cfg4["f"])
            r4["csr"] = csr_compare(c4, x4, 10, 3, dev)
            extras["c4_ms"] = r4["ms"]
            extras["c4"] = dict(r4, build=t4)
            del c4, x4
        else:
            c4, cfg4, t4, p4 = build_structure("c4", 1.0, build_device=local_rank)
            extras["c4"] = dict(sharded_spmm(c4, cfg4, "c4", 20, 5, dev, rank, world), build=t4)
            extras["c4_ms"] = extras["c4"]["ms"]
            del c4
            c5, cfg5, t5, p5 = build_structure("c5", 1.0, build_device=local_rank)
            extras["c5_gcn_forward"] = dict(sharded_gcn_forward(c5, cfg5, "c5", 5, 3, dev, rank, world), build=t5)
            extras["c5_gcn_forward_ms"] = extras["c5_gcn_forward"]["ms"]
            del c5
            dist.barrier()
            if rank == 0:
                for p in (p4, p5):
                    if os.path.exists(p):
                        os.unlink(p)
    bad = parity["max_err_over_tol"] > 1.0
    for v in extras.values():
        if isinstance(v, dict) and "parity" in v and v["parity"]["max_err_over_tol"] > 1.0:
            bad = True
    if rank == 0:
        line["extras"] = extras
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        if rank == 0 and os.path.exists(shared_path):
            os.unlink(shared_path)
        dist.destroy_process_group()
    if bad:
        sys.stderr.write("parity failure: an output element is outside atol + rtol |want|\n")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
