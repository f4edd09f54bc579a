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
        torch.manual_seed(0)
        model = ShardedGCN((100, 256, 47), sh).cuda()
        out = sh.from_labels(model(xl)).cpu().numpy()
        w1, w2 = (l.weight.detach().cpu().numpy().astype(np.float64) for l in model.lins)
        h = np.maximum(sparse_product(ei.numpy(), (x @ w1.T).astype(np.float32), True), 0)
        ref = sparse_product(ei.numpy(), (h @ w2.T).astype(np.float32), True)
        q.put((rank, err, float(np.abs(out - ref).max() / max(1.0, np.abs(ref).max()))))
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
