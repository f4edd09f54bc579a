"""Multi-GPU execution of the CBM product: whole subtrees of the virtual root per GPU.

The reference has no distributed code; its only parallel axis is "one subtree of the virtual root
per OpenMP task" (cbm/cbm_extensions.cpp:1168-1169).  The same unit is the shard here: a subtree's
rows depend only on each other and on the dense operand, so a GPU that owns whole subtrees needs no
data from its peers during the product.  Between two GCN layers every GPU needs all rows of the
layer output, which is one all-gather of row shards.

Vertices are relabelled so that each rank's rows are one contiguous block of ``shard_rows`` labels
(the last labels of a block are padding when the rank owns fewer rows).  With equal blocks the
all-gather is a single in-place ``all_gather_into_tensor`` over NCCL: every rank's kernel writes its
finished rows straight into its slice of the gathered buffer.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .cbm import _Plan, _as_f32, cbm_matrix


@dataclass
class Partition:
    perm: np.ndarray        # int32 [n]: label of every vertex
    n_labels: int           # world * shard_rows
    shard_rows: int         # labels per rank (multiple of 4 so shards stay 16-byte aligned)
    counts: np.ndarray      # rows actually owned by each rank
    cost: np.ndarray        # modelled work of each rank (delta entries + rows)
    world: int

    def offsets(self, rank: int) -> tuple[int, int]:
        return rank * self.shard_rows, (rank + 1) * self.shard_rows


def subtree_of_rows(c: cbm_matrix) -> np.ndarray:
    """For every row, the child of the virtual root whose subtree contains it."""
    n = c.num_rows
    parent = c._parent
    top = np.where(parent == n, np.arange(n, dtype=np.int64), -1)
    # rows in breadth-first order see their parent's entry already filled
    mr, mc = c.mst_row.numpy(), c.mst_col.numpy()
    frontier = mc[mr[n]:mr[n + 1]].astype(np.int64)
    while frontier.size:
        counts = (mr[frontier + 1] - mr[frontier]).astype(np.int64)
        if counts.sum() == 0:
            break
        starts = mr[frontier].astype(np.int64)
        idx = np.repeat(starts - np.concatenate([[0], np.cumsum(counts)[:-1]]), counts) + np.arange(counts.sum())
        children = mc[idx].astype(np.int64)
        top[children] = np.repeat(top[frontier], counts)
        frontier = children
    return top


def partition_subtrees(c: cbm_matrix, world: int) -> Partition:
    """Longest-processing-time packing of root subtrees onto ``world`` ranks.

    Cost of a subtree = its delta entries + its rows (one gathered operand row per entry, one
    stored row per row).  Ties go to the rank with fewer rows, which also evens out shard sizes.
    """
    n = c.num_rows
    top = subtree_of_rows(c)
    dlen = np.diff(c._crow).astype(np.int64)
    cost_of_top = np.bincount(top, weights=dlen + 1, minlength=n)
    rows_of_top = np.bincount(top, minlength=n)
    tops = np.nonzero(rows_of_top)[0]
    order = tops[np.lexsort((tops, -cost_of_top[tops]))]
    load = np.zeros(world)
    rows = np.zeros(world, dtype=np.int64)
    owner_of_top = np.full(n, -1, dtype=np.int64)
    n_head = min(order.size, 64 * world)
    for t in order[:n_head].tolist():  # exact greedy on the heavy subtrees
        g = int(np.lexsort((rows, load))[0])
        owner_of_top[t] = g
        load[g] += cost_of_top[t]
        rows[g] += rows_of_top[t]
    tail = order[n_head:]
    if tail.size:
        # the many light subtrees are dealt out in cost order, lightest rank first, reversing
        # direction every round so the ranks stay level
        k = np.arange(tail.size)
        rnd, pos = k // world, k % world
        slot = np.where(rnd % 2 == 0, pos, world - 1 - pos)
        owner_of_top[tail] = np.argsort(load, kind="stable")[slot]
        np.add.at(load, owner_of_top[tail], cost_of_top[tail])
        np.add.at(rows, owner_of_top[tail], rows_of_top[tail])
    owner = owner_of_top[top]
    counts = np.bincount(owner, minlength=world)
    shard_rows = int(-(-int(counts.max()) // 4) * 4)
    perm = np.empty(n, dtype=np.int32)
    for g in range(world):
        mine = np.nonzero(owner == g)[0]  # ascending original id keeps operand locality
        perm[mine] = g * shard_rows + np.arange(mine.size, dtype=np.int32)
    return Partition(perm=perm, n_labels=world * shard_rows, shard_rows=shard_rows, counts=counts,
                     cost=load, world=world)


class ShardedCBM:
    """One rank's share of a CBM product, plus the all-gather that completes a layer.

    ``group`` is a ``torch.distributed`` process group (NCCL on GPUs).  Dense tensors handled by
    this class live in LABEL space: ``to_labels`` / ``from_labels`` convert from / to the original
    vertex order once at the boundary of the model.
    """

    def __init__(self, c: cbm_matrix, rank: int, world: int, device_index: int | None = None, group=None,
                 partition: Partition | None = None):
        self.c, self.rank, self.world, self.group = c, rank, world, group
        self.part = partition or partition_subtrees(c, world)
        self.begin, self.end = self.part.offsets(rank)
        self.device_index = device_index
        self._plan = None
        self._perm_t = None

    @property
    def plan(self) -> _Plan:
        """Device schedule of this rank's rows (created on first use)."""
        if self._plan is None:
            c = self.c
            if self.device_index is None:
                self.device_index = torch.cuda.current_device()
            mul = None if c.col_multiplier is None else _as_f32(c.col_multiplier)
            self._plan = _Plan(c.num_rows, c.mst_row.numpy(), c.mst_col.numpy(), c._crow, c._dcol, c._dval, mul,
                               self.device_index, perm=self.part.perm, n_labels=self.part.n_labels,
                               own_begin=self.begin, own_end=self.end)
        return self._plan

    def _perm(self, device):
        if self._perm_t is None or self._perm_t.device != device:
            self._perm_t = torch.from_numpy(self.part.perm.astype(np.int64)).to(device)
        return self._perm_t

    def to_labels(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.zeros((self.part.n_labels, x.size(1)), dtype=x.dtype, device=x.device)
        out[self._perm(x.device)] = x
        return out

    def from_labels(self, y: torch.Tensor) -> torch.Tensor:
        return y[self._perm(y.device)]

    def local_product(self, x_labels: torch.Tensor, out_full: torch.Tensor) -> torch.Tensor:
        """Compute this rank's rows into its slice of ``out_full`` ([n_labels, F]) and return the slice."""
        from . import _lib
        import ctypes
        f = x_labels.size(1)
        mine = out_full[self.begin:self.end]
        fn = _lib.lib().cbm_b200_fused_spmm_update if self.c.normalized else _lib.lib().cbm_b200_spmm_update
        stream = torch.cuda.current_stream(x_labels.device).cuda_stream
        _lib.check(fn(self.plan.handle, x_labels.data_ptr(), x_labels.stride(0), mine.data_ptr(),
                      out_full.stride(0), f, ctypes.c_void_p(stream)))
        return mine

    def matmul(self, x_labels: torch.Tensor, gather: bool = True) -> torch.Tensor:
        """``A @ x`` in label space: local subtrees, then (optionally) the all-gather of shards.
        Padding labels of the result are zero."""
        out = torch.zeros((self.part.n_labels, x_labels.size(1)), dtype=x_labels.dtype, device=x_labels.device)
        mine = self.local_product(x_labels, out)
        if gather and self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(out, mine, group=self.group)
        return out


class ShardedGCN(torch.nn.Module):
    """Forward pass of a stack of GCN layers over a sharded CBM structure (weights replicated).

    Per layer and rank: the dense map ``lin`` on the rank's own block of rows (1/world of the
    GEMM), one in-place all-gather of the ``lin`` output shards (every rank needs all rows of the
    product's right-hand side), then the product over the rank's subtrees.  ReLU between layers is
    applied to the local block.  Everything lives in label space; padding rows are zero and stay
    zero because the layers have no bias.
    """

    def __init__(self, widths, sharded: ShardedCBM):
        super().__init__()
        self.sharded = sharded
        self._cache = {}
        self.lins = torch.nn.ModuleList(torch.nn.Linear(a, b, bias=False) for a, b in zip(widths[:-1], widths[1:]))
        for lin in self.lins:
            torch.nn.init.xavier_uniform_(lin.weight)

    def _work_buffers(self, width: int, like: torch.Tensor):
        """Two zero-initialised [n_labels, width] buffers per width, reused across calls: padding
        rows are never written, so they stay zero."""
        key = (width, like.device, like.dtype)
        if key not in self._cache:
            n = self.sharded.part.n_labels
            self._cache[key] = (torch.zeros((n, width), dtype=like.dtype, device=like.device),
                                torch.zeros((n, width), dtype=like.dtype, device=like.device))
        return self._cache[key]

    @torch.no_grad()
    def forward(self, x_labels: torch.Tensor, gather_output: bool = True) -> torch.Tensor:
        """``x_labels``: [n_labels, F_in] in label space.  Returns the output in label space
        (all rows when ``gather_output``, else only this rank's block is meaningful).  The returned
        tensor is a view of a buffer that the next call overwrites."""
        import torch.distributed as dist
        sh = self.sharded
        h_local = x_labels[sh.begin:sh.end]
        out = None
        for i, lin in enumerate(self.lins):
            if i:
                h_local = h_local.relu()
            f = lin.out_features
            fp = -(-f // 4) * 4  # widths are padded to a multiple of 4 floats for the 128-bit path
            z, out = self._work_buffers(fp, x_labels)
            prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = False  # full fp32, as the 1e-4 tolerance needs
            try:
                torch.mm(h_local[:, :lin.in_features], lin.weight.t(), out=z[sh.begin:sh.end, :f])
            finally:
                torch.backends.cuda.matmul.allow_tf32 = prev
            if sh.world > 1:
                dist.all_gather_into_tensor(z, z[sh.begin:sh.end], group=sh.group)
            h_local = sh.local_product(z, out)
        if gather_output and sh.world > 1:
            dist.all_gather_into_tensor(out, h_local, group=sh.group)
        return out[:, :self.lins[-1].out_features]
