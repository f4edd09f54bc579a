"""Sharded product and GCN forward on 2 GPUs (child processes, NCCL).  Skipped with fewer GPUs."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cbm4gnn_b200 import graphs
from cbm4gnn_b200.cbm import cbm_matrix
from cbm4gnn_b200.sharding import ShardedCBM, ShardedGCN
from cbm4gnn_b200.utility import add_self_loops
from helpers import sparse_product

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ei = add_self_loops(torch.from_numpy(graphs.make_graph("c1")))
        c = cbm_matrix(ei.to(torch.int32), torch.ones(ei.shape[1]), alpha=0, normalized=True)
        sh = ShardedCBM(c, rank, world, device_index=rank)
        n = c.num_rows
        x = graphs.make_features("c1", n, f=100)
        xl = sh.to_labels(torch.from_numpy(x).cuda())
        y = sh.from_labels(sh.matmul(xl)).cpu().numpy()
        sh.plan.status()
        err = float(np.abs(y - sparse_product(ei.numpy(), x, True)).max())
        err2 = 0.0
        # (100,256,47): propagate_first then lin_first; (100,64,96,47): lin_first -> propagate_first
        # -> lin_first, so with exchange="peer" one hand-over between layers and the model output
        # are delivered by the product kernel's stores into the peers' gathered buffers
        # (100,300,256,47): its 300 -> 256 layer is lin_first and wide, so dense map, all-gather and
        # product are pipelined over 128-column chunks
        for widths, exchange in (((100, 256, 47), "nccl"), ((100, 256, 47), "peer"), ((100, 64, 96, 47), "nccl"),
                                 ((100, 64, 96, 47), "peer"), ((100, 300, 256, 47), "nccl"), ((100, 300, 260, 47), "peer")):
            torch.manual_seed(0)
            model = ShardedGCN(widths, sh, exchange=exchange, pipeline_wide=len(widths) == 4).cuda()
            h = x.astype(np.float64)
            for k, l in enumerate(model.lins):
                w = l.weight.detach().cpu().numpy().astype(np.float64)
                h = sparse_product(ei.numpy(), (h @ w.T).astype(np.float32), True)
                if k < len(model.lins) - 1:
                    h = np.maximum(h, 0)
            for _ in range(2):  # buffers are reused between calls
                out = sh.from_labels(model(xl)).cpu().numpy()
            err2 = max(err2, float(np.abs(out - h).max() / max(1.0, np.abs(h).max())))
            par = model.check_last_product(xl, rows=200)
            err2 = max(err2, par["max_err_over_tol"] * 1e-4)
            assert len(model.timed_forward(xl)) == len(widths) - 1
        # operands in host memory: own block over PCIe, all-gather over NVLink, product, copy back
        xh = xl.cpu().pin_memory()
        yh = torch.empty((sh.part.shard_rows, 100)).pin_memory()
        full = sh.matmul(xl)
        for chunk in (128, 32):  # one chunk, and four pipelined chunks
            yh.fill_(float("nan"))
            sh.host_product(xh[sh.begin:sh.end], yh, chunk=chunk)
            torch.testing.assert_close(yh, full[sh.begin:sh.end].cpu(), atol=1e-5, rtol=1e-5)
        q.put((rank, err, err2))
    finally:
        dist.destroy_process_group()


def test_two_gpus_sharded_product_and_gcn_forward():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 400
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, err, err2 in res:
        assert err < 1e-4 and err2 < 1e-4, (rank, err, err2)
