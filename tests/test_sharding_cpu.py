"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world_size 2): subtree partition,
label bookkeeping and the in-place all-gather.  The per-rank product is computed by the CPU
restatement here (there is no GPU); the CUDA plans of a shard are covered by the GPU tests."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cbm4gnn_b200 import graphs
from cbm4gnn_b200.cbm import cbm_matrix
from cbm4gnn_b200.sharding import ShardedCBM, ShardedGCN, partition_subtrees, subtree_of_rows
from cbm4gnn_b200.utility import add_self_loops
from oracle import cbm_oracle as orc
from helpers import sparse_product


def _structure(scale=0.25, alpha=0):
    ei = add_self_loops(torch.from_numpy(graphs.make_graph("c1", scale=scale)))
    return ei, cbm_matrix(ei.to(torch.int32), torch.ones(ei.shape[1]), alpha=alpha, normalized=True)


@pytest.mark.parametrize("world", [2, 3, 8])
def test_partition_owns_whole_subtrees_and_balances(world):
    _, c = _structure(1.0)
    part = partition_subtrees(c, world)
    n = c.num_rows
    assert sorted(part.perm.tolist()) == sorted(set(part.perm.tolist())) and part.perm.max() < part.n_labels
    owner = part.perm // part.shard_rows
    parent = c._parent
    inner = parent != n
    assert np.array_equal(owner[inner], owner[parent[inner]])          # no subtree is cut
    assert part.counts.sum() == n and part.shard_rows % 4 == 0
    assert np.array_equal(np.bincount(owner, minlength=world), part.counts)
    assert part.cost.max() <= 1.25 * part.cost.mean()                   # LPT keeps the ranks level
    top = subtree_of_rows(c)
    assert np.array_equal(top[inner], top[parent[inner]]) and np.all(parent[top] == n)


class _OracleShard(ShardedCBM):
    """Per-rank product through the CPU restatement instead of a CUDA plan."""

    def product_into(self, x_labels, y_shard, bcast=None, relu=False):
        c = self.c
        x = x_labels[torch.from_numpy(self.part.perm.astype(np.int64))].numpy()   # back to vertex order
        y = orc.fused_spmm_update(c.mst_row.numpy(), c.mst_col.numpy(), c._crow, c._dcol, c._dval,
                                  c.col_multiplier.numpy(), np.ascontiguousarray(x), parallel=False)
        lab = self.part.perm
        own = (lab >= self.begin) & (lab < self.end)
        y_shard[torch.from_numpy(lab[own] - self.begin).long()] = torch.from_numpy(y[own])
        return y_shard


def _worker(rank, world, port, fail_rank, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ei, c = _structure()
        sh = _OracleShard(c, rank, world)
        n = c.num_rows
        x = graphs.make_features("c1", n, f=12)
        xl = sh.to_labels(torch.from_numpy(x))
        y = sh.from_labels(sh.matmul(xl)).numpy()
        err = float(np.abs(y - sparse_product(ei.numpy(), x, True)).max())
        # two stacked layers in label space equal the unsharded computation
        # widths chosen so that both layer orders and both hand-overs between them occur:
        # (12,16,5) = propagate_first then lin_first, (12,8,10,10) = lin_first, propagate_first, lin_first
        err2 = 0.0
        for widths in ((12, 16, 5), (12, 8, 10, 10)):
            torch.manual_seed(0)
            model = ShardedGCN(widths, sh)
            assert model.orders == ["propagate_first" if a < b else "lin_first" for a, b in zip(widths[:-1], widths[1:])]
            out = sh.from_labels(model(xl)).numpy()
            h = x
            for k, l in enumerate(model.lins):
                w = l.weight.detach().numpy().astype(np.float64)
                h = sparse_product(ei.numpy(), (h @ w.T).astype(np.float32), True)
                if k < len(model.lins) - 1:
                    h = np.maximum(h, 0)
            err2 = max(err2, float(np.abs(out - h).max()))
            # without the final gather the rank's own block is still right
            own = (sh.part.perm >= sh.begin) & (sh.part.perm < sh.end)
            loc = sh.from_labels(model(xl, gather_output=False)).numpy()
            err2 = max(err2, float(np.abs(loc[own] - h[own]).max()))
        q.put((rank, err, err2))
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_reproduce_the_full_product():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, -1, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, err2 in res:
        assert err < 1e-4 and err2 < 1e-3, (rank, err, err2)
