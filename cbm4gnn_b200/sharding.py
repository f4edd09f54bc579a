"""Multi-GPU execution of the CBM product: whole subtrees of the virtual root per GPU.

The reference has no distributed code; its only parallel axis is "one subtree of the virtual root
per OpenMP task" (cbm/cbm_extensions.cpp:1168-1169).  The same unit is the shard here: a subtree's
rows depend only on each other and on the dense operand, so a GPU that owns whole subtrees needs no
data from its peers during the product.  Between two GCN layers every GPU needs all rows of the
layer output, which is one all-gather of row shards.

Vertices are relabelled so that each rank's rows are one contiguous block of ``shard_rows`` labels
(the last labels of a block are padding when the rank owns fewer rows).  With equal blocks the
all-gather is a single in-place ``all_gather_into_tensor`` over NCCL: every rank's kernel writes its
finished rows straight into its slice of the gathered buffer.  Where a product's output is what
the next product gathers (or the model's output), the exchange can instead be done by the product
kernel itself: every finished row is stored into the slice this shard occupies in every GPU's copy
of the gathered buffer (peer memory reached by ordinary stores over NVLink), so the transfer runs
while the product runs, followed by one barrier.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .cbm import _Plan, _as_f32, aligned_rows, cbm_matrix


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
        self._host_bufs = {}

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
        """``x`` (vertex order) as a label-space operand: padding labels zero, rows pitched to whole
        128-byte lines (see ``aligned_rows``)."""
        out = aligned_rows(self.part.n_labels, x.size(1), x.device, x.dtype)
        out[self._perm(x.device)] = x
        return out

    def from_labels(self, y: torch.Tensor) -> torch.Tensor:
        return y[self._perm(y.device)]

    def product_into(self, x_labels: torch.Tensor, y_shard: torch.Tensor, bcast=None, relu: bool = False) -> torch.Tensor:
        """This rank's rows of the product into ``y_shard`` ([shard_rows, F], any row stride).
        ``bcast``: device addresses (this GPU's or peers') of further buffers with ``y_shard``'s
        layout that receive every finished row as it is produced, after a ReLU when ``relu``."""
        from . import _lib
        import ctypes
        f = x_labels.size(1)
        L = _lib.lib()
        stream = ctypes.c_void_p(torch.cuda.current_stream(x_labels.device).cuda_stream)
        if bcast:
            arr = (ctypes.c_void_p * len(bcast))(*bcast)
            _lib.check(L.cbm_b200_spmm_update_bcast(self.plan.handle, x_labels.data_ptr(), x_labels.stride(0),
                                                    y_shard.data_ptr(), y_shard.stride(0), f,
                                                    1 if self.c.normalized else 0, 1 if relu else 0, len(bcast),
                                                    arr, stream))
        else:
            fn = L.cbm_b200_fused_spmm_update if self.c.normalized else L.cbm_b200_spmm_update
            _lib.check(fn(self.plan.handle, x_labels.data_ptr(), x_labels.stride(0), y_shard.data_ptr(),
                          y_shard.stride(0), f, stream))
        return y_shard

    def local_product(self, x_labels: torch.Tensor, out_full: torch.Tensor) -> torch.Tensor:
        """Compute this rank's rows into its slice of ``out_full`` ([n_labels, F]) and return the slice."""
        return self.product_into(x_labels, out_full[self.begin:self.end])

    def matmul(self, x_labels: torch.Tensor, gather: bool = True) -> torch.Tensor:
        """``A @ x`` in label space: local subtrees, then (optionally) the all-gather of shards.
        Padding labels of the result are zero."""
        out = torch.zeros((self.part.n_labels, x_labels.size(1)), dtype=x_labels.dtype, device=x_labels.device)
        mine = self.local_product(x_labels, out)
        if gather and self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(out, mine, group=self.group)
        return out

    def host_product(self, x_mine_host: torch.Tensor, y_host: torch.Tensor, chunk: int = 128) -> None:
        """The product for operands that live in host memory, one block of rows per rank.

        ``x_mine_host``: this rank's block of the operand, [shard_rows, F] in label space,
        contiguous (pinned memory makes the copies asynchronous); ``y_host``: [shard_rows, F]
        contiguous, receives this rank's rows of the result.  Pipelined over column chunks: each rank
        sends only its own block of a chunk over PCIe, one all-gather over NVLink completes the chunk
        on every GPU, the product of the chunk runs and its result goes back — while the next chunk
        is already on its way in (PCIe is full duplex).  Returns when ``y_host`` is complete."""
        import ctypes
        import torch.distributed as dist
        from . import _lib
        L = _lib.lib()
        if not (x_mine_host.is_contiguous() and y_host.is_contiguous()):
            raise RuntimeError("host operands must be contiguous")
        f = int(x_mine_host.size(1))
        rows = self.part.shard_rows
        dev = torch.device("cuda", self.plan.device_index)
        cols = [(c0, min(chunk, f - c0)) for c0 in range(0, f, chunk)]
        key = (f, chunk)
        st = self._host_bufs.get(key)
        if st is None:
            st = dict(xc=[torch.zeros((self.part.n_labels, w), device=dev) for _, w in cols],
                      y=aligned_rows(rows, f, dev), cin=torch.cuda.Stream(dev), comm=torch.cuda.Stream(dev),
                      cout=torch.cuda.Stream(dev))
            self._host_bufs = {key: st}
        cur = torch.cuda.current_stream(dev)
        start = torch.cuda.Event()
        start.record(cur)
        st["cin"].wait_event(start)      # earlier work on the caller's stream (and the last call) is done
        xp, yp = x_mine_host.data_ptr(), y_host.data_ptr()
        for k, (c0, w) in enumerate(cols):
            xc = st["xc"][k]
            mine = xc[self.begin:self.end]
            _lib.check(L.cbm_b200_copy2d_async(ctypes.c_void_p(mine.data_ptr()), w * 4, ctypes.c_void_p(xp + c0 * 4), f * 4,
                                               w * 4, rows, 1, ctypes.c_void_p(st["cin"].cuda_stream)))
            arrived = torch.cuda.Event()
            arrived.record(st["cin"])
            gathered = arrived
            if self.world > 1:
                with torch.cuda.stream(st["comm"]):
                    st["comm"].wait_event(arrived)
                    dist.all_gather_into_tensor(xc, mine, group=self.group)
                    gathered = torch.cuda.Event()
                    gathered.record(st["comm"])
            cur.wait_event(gathered)
            self.product_into(xc, st["y"][:, c0:c0 + w])
            done = torch.cuda.Event()
            done.record(cur)
            st["cout"].wait_event(done)
            _lib.check(L.cbm_b200_copy2d_async(ctypes.c_void_p(yp + c0 * 4), f * 4, ctypes.c_void_p(st["y"].data_ptr() + c0 * 4),
                                               st["y"].stride(0) * 4, w * 4, rows, 0, ctypes.c_void_p(st["cout"].cuda_stream)))
        st["cout"].synchronize()


class PeerBuffer:
    """A [n_labels, width] buffer that exists at the same size on every rank with every rank's
    copy mapped into every process (``torch.distributed._symmetric_memory``): the gathered layer
    output that the product kernels of all GPUs write into directly."""

    def __init__(self, n_labels: int, width: int, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.tensor = symm_mem.empty((n_labels, width), dtype=torch.float32, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.row_bytes = width * 4

    def slice_addresses(self, first_row: int) -> list[int]:
        """Device address of row ``first_row`` in every rank's copy (own copy included)."""
        return [p + first_row * self.row_bytes for p in self.ptrs]

    def barrier(self):
        """All ranks' earlier stores into all copies are complete and visible after this."""
        self.handle.barrier(channel=0)


class ShardedGCN(torch.nn.Module):
    """Forward pass of a stack of GCN layers over a sharded CBM structure (weights replicated).

    Per layer and rank, in the cheaper of two equivalent orders (``A (H W) = (A H) W``):
    * "lin_first" (the reference's order, cbm_gcn.py:21-24; chosen when in >= out): the dense map
      on the rank's own rows, an exchange of its output (every rank needs all rows of the
      product's right-hand side), the product over the rank's subtrees;
    * "propagate_first" (in < out): an exchange of the layer input, the product at the input
      width, the dense map on the rank's own rows.
    ``pipeline_wide``: lin_first layers of 256 columns and more run in 128-column chunks, dense map
    and all-gather of the next chunk (side stream) under the product of the current one.  Measured on
    the 2.4 M-node block-model graph the 256-wide layer goes from 8.8 to 8.2 ms on 2 GPUs but from
    5.05 to 5.36 ms on 8 (the all-gather and the product slow each other down), so it is off by default.
    ReLU between layers acts on the local block.  ``exchange``: "nccl" = in-place
    ``all_gather_into_tensor``; "peer" = where the exchanged tensor is a product's output (a
    lin_first layer followed by a propagate_first layer, and the gathered model output) the
    product kernel stores finished rows straight into every GPU's gathered buffer, ReLU applied
    on the way, followed by one barrier; other exchanges stay on NCCL.
    Everything lives in label space; padding rows are zero and stay zero (no bias).
    """

    def __init__(self, widths, sharded: ShardedCBM, exchange: str = "nccl", pipeline_wide: bool = False):
        super().__init__()
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.sharded = sharded
        self.pipeline_wide = pipeline_wide
        self.exchange = exchange if sharded.world > 1 else "nccl"
        self._cache = {}
        self._peer = {}
        self.lins = torch.nn.ModuleList(torch.nn.Linear(a, b, bias=False) for a, b in zip(widths[:-1], widths[1:]))
        for lin in self.lins:
            torch.nn.init.xavier_uniform_(lin.weight)
        self.orders = ["propagate_first" if lin.in_features < lin.out_features else "lin_first" for lin in self.lins]

    def _buffer(self, tag: str, width: int, like: torch.Tensor, rows: int | None = None):
        """Zero-initialised work buffer, reused across calls (padding rows are never written, so
        they stay zero)."""
        rows = self.sharded.part.n_labels if rows is None else rows
        key = (tag, width, rows, like.device)
        if key not in self._cache:
            self._cache[key] = torch.zeros((rows, width), dtype=torch.float32, device=like.device)
        return self._cache[key]

    def _peer_buffer(self, tag: str, width: int, like: torch.Tensor) -> PeerBuffer:
        key = (tag, width)
        if key not in self._peer:
            self._peer[key] = PeerBuffer(self.sharded.part.n_labels, width, like.device, self.sharded.group)
        return self._peer[key]

    @staticmethod
    def _mm(h, lin, out, relu=False):
        """``out = h @ lin.weight.T`` (``relu``: then ``max(., 0)``) in fp32 accuracy (tensor-core
        GEMM on CUDA tensors, the ReLU in its epilogue)."""
        if h.is_cuda:
            from .dense import dense_forward
            dense_forward(h, lin.weight, out=out, relu=relu)
        else:
            torch.mm(h, lin.weight.t(), out=out)
            if relu:
                out.relu_()

    @staticmethod
    def _mm_rows(h, w_rows, out):
        """``out = h @ w_rows.T`` for a block of weight rows (a column chunk of the layer's output)."""
        if h.is_cuda:
            from .dense import dense_forward
            dense_forward(h, w_rows, out=out)
        else:
            torch.mm(h, w_rows.t(), out=out)

    def _side_stream(self, device):
        if getattr(self, "_comm_stream", None) is None:
            self._comm_stream = torch.cuda.Stream(device=device)
        return self._comm_stream

    def _gather(self, full, mine):
        import torch.distributed as dist
        if self.sharded.world > 1:
            dist.all_gather_into_tensor(full, mine, group=self.sharded.group)

    @torch.no_grad()
    def forward(self, x_labels: torch.Tensor, gather_output: bool = True, probe: dict | None = None) -> torch.Tensor:
        """``x_labels``: [n_labels, F_in] in label space, all rows present on every rank.  Returns
        the output in label space (all rows when ``gather_output``, else only this rank's block is
        meaningful).  The returned tensor is a view of a buffer that the next call overwrites.
        ``probe`` (a dict) receives per-layer phase times in ms and the last product's operands."""
        sh = self.sharded
        n_layers = len(self.lins)
        timing = probe is not None

        def tick():
            if not timing:
                return None
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e

        phases = []
        h_full = x_labels                      # all rows of the current layer input, or None
        h_local = x_labels[sh.begin:sh.end]    # this rank's rows of it
        y_full = None
        for i, lin in enumerate(self.lins):
            a, b = lin.in_features, lin.out_features
            bp = -(-b // 4) * 4
            last = i == n_layers - 1
            # will whoever consumes this layer's output need all rows of it on every rank?
            next_gathers = (not last and self.orders[i + 1] == "propagate_first") or (last and gather_output)
            y_full = self._buffer("y%d" % i, bp, x_labels)
            y_local = y_full[sh.begin:sh.end]
            delivered = False
            t0 = tick()
            if self.orders[i] == "propagate_first":
                ap = -(-a // 4) * 4
                if h_full is None:
                    h_full = self._buffer("hin%d" % i, ap, x_labels)
                    mine = h_full[sh.begin:sh.end]
                    mine[:, :a].copy_(h_local[:, :a])
                    self._gather(h_full, mine)
                elif h_full.size(1) != ap or h_full.stride(0) % 4:
                    padded = self._buffer("hpad%d" % i, ap, x_labels)
                    padded[:, :a].copy_(h_full[:, :a])
                    h_full = padded
                t1 = tick()
                p_local = self._buffer("p%d" % i, ap, x_labels, rows=sh.part.shard_rows)
                sh.product_into(h_full, p_local)
                t2 = tick()
                self._mm(p_local[:, :a], lin, y_local[:, :b], relu=not last)
                t3 = tick()
                kinds, prod = ("exchange", "product", "dense"), (h_full, p_local, ap)
            elif (self.pipeline_wide and sh.world > 1 and bp >= 256 and x_labels.is_cuda
                  and not (next_gathers and self.exchange == "peer")):
                # Wide lin_first layer: the dense map, its all-gather and the product all work on
                # independent 128-column chunks, so chunk k+1 is mapped and gathered (on a side
                # stream) while the product of chunk k runs.  Each chunk is its own contiguous
                # [n_labels, 128] buffer, which the in-place all-gather needs.
                import torch.distributed as dist
                cur = torch.cuda.current_stream(x_labels.device)
                comm = self._side_stream(x_labels.device)
                cols = [(c0, min(128, bp - c0)) for c0 in range(0, bp, 128)]
                zc, done = [], []
                for k, (c0, w) in enumerate(cols):
                    z = self._buffer("zc%d_%d" % (i, k), w, x_labels)
                    zc.append(z)
                    wr = min(w, b - c0)  # real (unpadded) columns of this chunk
                    self._mm_rows(h_local[:, :a], lin.weight[c0:c0 + wr], z[sh.begin:sh.end, :wr])
                    ready = torch.cuda.Event()
                    ready.record(cur)
                    with torch.cuda.stream(comm):
                        comm.wait_event(ready)
                        dist.all_gather_into_tensor(z, z[sh.begin:sh.end], group=sh.group)
                        ev = torch.cuda.Event()
                        ev.record(comm)
                        done.append(ev)
                t1 = tick()
                cur.wait_event(done[0])
                t2 = tick()
                for k, (c0, w) in enumerate(cols):
                    cur.wait_event(done[k])
                    sh.product_into(zc[k], y_local[:, c0:c0 + w])
                prod = (None, None, bp)
                if timing and last:
                    z_all = torch.cat(zc, dim=1)
                    prod = (z_all, y_local.clone(), bp)
                if not last:
                    y_local.relu_()
                t3 = tick()
                kinds = ("dense", "exchange", "product")
            else:
                z_full = self._buffer("z%d" % i, bp, x_labels)
                self._mm(h_local[:, :a], lin, z_full[sh.begin:sh.end, :b])
                t1 = tick()
                self._gather(z_full, z_full[sh.begin:sh.end])
                t2 = tick()
                if next_gathers and self.exchange == "peer":
                    # the product's output is what gets exchanged next: the kernel delivers it
                    pb = self._peer_buffer("g%d" % i, bp, x_labels)
                    pb.barrier()                       # every rank is done reading the previous contents
                    raw = self._buffer("raw%d" % i, bp, x_labels, rows=sh.part.shard_rows)
                    sh.product_into(z_full, raw, bcast=pb.slice_addresses(sh.begin), relu=not last)
                    pb.barrier()
                    y_full, y_local, delivered = pb.tensor, pb.tensor[sh.begin:sh.end], True
                    prod = (z_full, raw if last else None, bp)
                else:
                    sh.product_into(z_full, y_local)
                    prod = (z_full, y_local.clone() if (timing and last) else None, bp)
                    if not last:
                        y_local.relu_()
                t3 = tick()
                kinds = ("dense", "exchange", "product")
            if timing:
                phases.append(dict(order=self.orders[i], product_width=prod[2], exchange_width=prod[2],
                                   ev=(t0, t1, t2, t3), kinds=kinds))
                if last:
                    probe["last_product"] = prod
            h_local, h_full = y_local, None
            if delivered:
                h_full = y_full
            elif next_gathers:
                self._gather(y_full, y_local)
                h_full = y_full
        if timing:
            torch.cuda.synchronize()
            rows = []
            for ph in phases:
                t = ph.pop("ev")
                kinds = ph.pop("kinds")
                d = dict(ph, product_ms=0.0, exchange_ms=0.0, dense_ms=0.0)
                for k, (e0, e1) in zip(kinds, zip(t[:-1], t[1:])):
                    d[k + "_ms"] = e0.elapsed_time(e1)
                rows.append(d)
            probe["phases"] = rows
        return y_full[:, :self.lins[-1].out_features]

    def timed_forward(self, x_labels: torch.Tensor) -> list[dict]:
        """One forward pass with device timestamps between the phases of every layer.  In a
        lin_first layer delivered by the product kernel ("peer"), the exchange of its output is
        inside ``product_ms``."""
        probe: dict = {}
        self.forward(x_labels, gather_output=False, probe=probe)
        return probe["phases"]

    def check_last_product(self, x_labels: torch.Tensor, rows: int = 500) -> dict:
        """Sampled rows this rank owns of the LAST layer's sparse product, given the operand the
        model itself fed it, against a float64 CSR product on the host."""
        sh, c = self.sharded, self.sharded.c
        probe: dict = {}
        self.forward(x_labels, gather_output=False, probe=probe)
        operand, result, width = probe["last_product"]
        lab = sh.part.perm
        own = np.nonzero((lab >= sh.begin) & (lab < sh.end))[0]
        pick = np.sort(np.random.default_rng(77 + sh.rank).choice(own, min(rows, own.size), replace=False))
        x_vertex = operand[sh._perm(operand.device)].cpu().numpy().astype(np.float64)   # label -> vertex order
        got = result[torch.from_numpy((lab[pick] - sh.begin).astype(np.int64)).to(result.device)].cpu().numpy()
        keep = np.isin(c._row, pick)
        import scipy.sparse as sp
        n = c.num_rows
        sub = sp.csr_matrix((np.ones(int(keep.sum())), (c._row[keep], c._col[keep])), shape=(n, n))[pick]
        if c.col_multiplier is not None:
            s = c.col_multiplier.numpy().astype(np.float64)
            sub = sp.diags(s[pick]) @ sub @ sp.diags(s)
        want = np.asarray(sub @ x_vertex)
        d = np.abs(got.astype(np.float64) - want)
        return dict(rows=int(pick.size), max_abs_err=float(d.max()),
                    max_rel_err=float(d.max() / max(1e-30, np.abs(want).max())),
                    max_err_over_tol=float((d / (1e-4 + 1e-4 * np.abs(want))).max()))
