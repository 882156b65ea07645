"""Row-range sharding of fused-rowwise embedding tables over the GPUs of one node.

A table too large for one device is cut into contiguous row ranges, rank g holding rows
[g*R/G, (g+1)*R/G).  Every rank sees the whole request (lengths, indices, weights number the
whole table), pools the rows it owns -- the gather-pool kernel skips the others -- and the fp32
partial sums of the G ranks are added and rounded once to the result type, so the sharded
operator keeps the accumulation precision of the whole one; only the order of the fp32 additions
differs.  The batch is split over the ranks for the result: rank h ends with bags
[h*B/G, (h+1)*B/G) of every table.

Glow itself never splits an embedding table by rows (its ParallelTransformKind splits
SparseLengthsSum by batch only, lib/Optimizer/GraphOptimizer/GraphOptimizer.cpp:7263-7300);
the exchange here plays the part of a reduce-scatter over the batch dimension.

Exchange modes:
  "fused": the pooling kernel stores each partial bag straight into the slab of the rank that
           owns the bag (peer stores over NVLink), a one-element all-reduce on the stream is the
           rendezvous, then one kernel adds the G slabs;
  "nccl" : partials land in a local buffer, ncclReduceScatter adds them (the library baseline);
  "local": one rank, no exchange;
  "emulated": several ranks as objects of one process on one GPU (tests): the slabs are plain
           tensors, `pool` of every rank runs before `reduce` of any.
"""
import numpy as np
import torch

from . import ops


def row_range(rank, world, rows):
    """Rows [lo, hi) of a table of `rows` rows that rank `rank` of `world` holds."""
    return rank * rows // world, (rank + 1) * rows // world


def bag_range(rank, world, bags):
    """Bags [lo, hi) whose results rank `rank` ends up with (bags must divide evenly)."""
    if bags % world:
        raise ValueError("the number of bags (%d) must be a multiple of the number of ranks (%d)" % (bags, world))
    per = bags // world
    return rank * per, (rank + 1) * per


def bucketize(lengths, indices, weights, lo, hi):
    """The request cut down to rows [lo, hi): per-bag lengths, LOCAL row numbers (index - lo) and
    weights of the entries that fall in the range, in their order.  This is the host-side form of
    what the kernel's row-range filter does on the fly; a front end that routes indices to the
    owning GPU sends exactly these arrays."""
    lengths = np.asarray(lengths, np.int64)
    n = int(lengths.sum())
    idx = np.asarray(indices[:n])
    keep = (idx >= lo) & (idx < hi)
    bag_of = np.repeat(np.arange(len(lengths)), lengths)
    sub_len = np.bincount(bag_of[keep], minlength=len(lengths)).astype(np.int32)
    return sub_len, (idx[keep] - lo).astype(idx.dtype), np.asarray(weights[:n])[keep]


class RowShardedSLWS:
    """FusedRowwiseQuantizedSparseLengthsWeightedSum over T row-range sharded tables.

    shards: this rank's row ranges of the tables (CUDA uint8 [rows_of_shard, in_line] each);
    total_rows: rows of each whole table.  The result of `run` is this rank's [T, B/G, D] slice,
    in `out_dtype` (fp16 for the FP16 fused kinds unless stated).
    """

    def __init__(self, kind, shards, total_rows, batch, rank=0, world=1, group=None, exchange=None, out_dtype=None):
        self.kind, self.shards, self.total_rows = kind, list(shards), list(total_rows)
        self.rank, self.world, self.group = rank, world, group
        self.exchange = exchange or ("fused" if world > 1 else "local")
        if self.exchange not in ("fused", "nccl", "local", "emulated") or (world > 1) == (self.exchange == "local"):
            raise ValueError("exchange %r does not fit %d ranks" % (self.exchange, world))
        self.device = self.shards[0].device
        self.in_line = int(self.shards[0].shape[1])
        self.D = ops.out_columns(self.in_line, kind)
        self.batch = batch
        self.per = bag_range(0, world, batch)[1]
        self.out_dtype = out_dtype or ops.result_dtype(kind)
        self.row_ranges = [(row_range(rank, world, r)[0], r) for r in self.total_rows]
        for s, (lo, r) in zip(self.shards, self.row_ranges):
            if s.shape[0] != row_range(rank, world, r)[1] - lo:
                raise ValueError("shard holds %d rows, its range has %d" % (s.shape[0], row_range(rank, world, r)[1] - lo))
        T = len(self.shards)
        slab_bytes = world * T * self.per * self.D * 4
        if self.exchange == "fused":
            self.slab_buf = [ops.PeerBuffer(slab_bytes) for _ in range(2)]
            self.slabs = [b.as_tensor((world, T, self.per, self.D), torch.float32) for b in self.slab_buf]
            self.token = torch.zeros(1, dtype=torch.float32, device=self.device)
            self.peers = None
        else:
            self.slabs = [torch.empty((world, T, self.per, self.D), dtype=torch.float32, device=self.device)]
            self.peers = None
        if self.exchange == "nccl":
            self.reduced = torch.empty((T, self.per, self.D), dtype=torch.float32, device=self.device)
        self.out = torch.empty((T, self.per, self.D), dtype=self.out_dtype, device=self.device)
        self.status = ops.new_status(self.device)
        self.step = 0

    def connect_peers(self):
        """fused exchange: swap the IPC handles of the receive slabs with every rank."""
        import torch.distributed as dist
        handles = [None] * self.world
        dist.all_gather_object(handles, [b.handle for b in self.slab_buf], group=self.group)
        self.peers = [[self.slab_buf[s].ptr if r == self.rank else self.slab_buf[s].open(handles[r][s])
                       for r in range(self.world)] for s in range(2)]

    def set_peers(self, ranks):
        """emulated exchange: every rank's slab is a plain tensor of this process."""
        self.peers = [[r.slabs[0].data_ptr() for r in ranks]]

    def release(self):
        if self.exchange == "fused":
            for b in self.slab_buf:
                b.release()

    def prepare(self, weights, indices, lengths, slab=0, routed=False):
        """Binds one request (lists over the tables; fp32 weights -- an fp16 weight widened is the
        same number -- int64/int32 indices of the WHOLE table, int32 lengths [batch]) to receive
        slab `slab`.  routed=True: the request was already cut down to this rank's rows by the
        front end (`bucketize`: local row numbers, per-bag counts of this shard), so the kernel
        has nothing to skip."""
        T, per, D = len(self.shards), self.per, self.D
        by_source = self.exchange in ("fused", "emulated")
        if by_source:
            if self.peers is None:
                raise RuntimeError("connect_peers() / set_peers() has not run")
            bases = self.peers[slab]
        else:
            bases = [self.slabs[0].data_ptr()] * self.world
        # rank h's slab is [source rank, table, bag, column]; with a local buffer the "source"
        # axis is the destination chunk instead (the layout ncclReduceScatter wants)
        scatter = []
        for t in range(T):
            if by_source:
                scatter.append([bases[h] + ((self.rank * T + t) * per * D) * 4 for h in range(self.world)])
            else:
                scatter.append([bases[h] + ((h * T + t) * per * D) * 4 for h in range(self.world)])
        b = ops.SlwsBatch(self.kind, self.in_line, indices[0].dtype, device=self.device)
        b.bind(self.shards, weights, indices, lengths, None, dest_stride=D, scatter=scatter, bags_per_dest=per,
               row_ranges=None if routed else self.row_ranges)
        return b

    def pool(self, bound):
        """emulated exchange, first half: this rank's partial bags into every rank's slab."""
        bound.run(self.status)

    def reduce(self):
        """emulated exchange, second half: add the slabs the ranks filled."""
        return ops.sum_partials(self.slabs[0].view(self.world, -1), out=self.out)

    def run(self, bound_pair):
        """bound_pair[slab]: the request bound to each receive slab (one entry unless fused)."""
        slab = (self.step & 1) if self.exchange == "fused" else 0
        if self.exchange == "emulated":
            raise RuntimeError("emulated ranks run pool() on every rank, then reduce()")
        bound_pair[slab].run(self.status)
        if self.exchange == "fused":
            import torch.distributed as dist
            dist.all_reduce(self.token, group=self.group)  # every rank's peer stores are complete after it
            ops.sum_partials(self.slabs[slab].view(self.world, -1), out=self.out)
        elif self.exchange == "nccl":
            import torch.distributed as dist
            dist.reduce_scatter_tensor(self.reduced, self.slabs[0], group=self.group)
            ops.sum_partials(self.reduced.view(1, -1), out=self.out)
        else:
            ops.sum_partials(self.slabs[0].view(1, -1), out=self.out)
        self.step += 1
        return self.out

    def run_request(self, weights, indices, lengths):
        slab = (self.step & 1) if self.exchange == "fused" else 0
        pair = [None, None]
        pair[slab] = self.prepare(weights, indices, lengths, slab)
        return self.run(pair)
