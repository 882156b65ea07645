"""DLRM-style recommendation model on the glow_b200 kernels (benchmark configuration 4).

    dense fp32 [B,256] -> Quantize -> bottom MLP (int8 rowwise FC + Relu) -> Dequantize -> x0 [B,128]
    T tables, fused-rowwise uint8 [rows, 128+8]  -> SparseLengthsSum per table    -> pooled [B,T,128]
    interaction: [x0 | dot(v_i, v_j), j < i over the T+1 vectors] -> Quantize      -> [B,128 + (T+1)T/2]
    top MLP (int8 rowwise FC + Relu, last layer linear) -> Dequantize              -> [B,1]

The graph is the one tests/unittests/RecommendationSystemTest.cpp:872-950 builds (with the
strictly-lower-triangle interaction the benchmark configuration asks for).  Across G GPUs the
tables are sharded by table (Glow's SparseNN partitioner, lib/Partitioner/Partitioner.cpp:
1611-1685): every rank pools ITS tables for the WHOLE batch, the pooled vectors are exchanged so
that rank r ends up with [B/G, T, D] for ITS slice of the batch, and the dense layers run
batch-sharded.  Two forms of the exchange exist:
  * "nccl":  pool into a local [G, B/G, T_local, D] buffer, torch.distributed.all_to_all_single;
  * "fused": the pooling kernel stores every bag straight into the destination rank's
             [B/G, T, D] slab through peer pointers (NVLink stores), followed by a barrier.

This module is harness code (model building, calibration, request plumbing).  All arithmetic
that reaches the result runs in the CUDA library, through glow_b200.ops.
"""
import math
from dataclasses import dataclass, field

import numpy as np
import torch

from . import ops


@dataclass
class DLRMConfig:
    tables: int = 64
    rows: int = 4_000_000
    dim: int = 128
    batch: int = 4096
    dense_in: int = 256
    bottom: tuple = (512, 256, 128)
    top: tuple = (1024, 1024, 512, 1)
    mean_len: float = 40.0
    max_len: int = 200
    zipf_s: float = 1.05
    seed: int = 0x610B200
    # Schema of the rowwise-quantized MLP weights (the `schema` argument of
    # Function::createRowwiseQuantizedFullyConnected, lib/Graph/Graph.cpp:1198-1246).  Symmetric
    # rows have offset 0, which takes the activation row sums (one more pass over every layer's
    # input) out of the step; He-normal weights are centred, so the ranges lose next to nothing.
    weights_schema: str = "symmetric"

    @property
    def interaction_width(self):
        n = self.tables + 1
        return self.dim + n * (n - 1) // 2


# ------------------------------------------------------------------------------------------
# synthetic data (seeded; same laws on numpy and on torch/cuda)
# ------------------------------------------------------------------------------------------
def _zipf_rank(u, n, s):
    """Inverse CDF of a continuous power law on [1, n+1): rank-1 in [0, n)."""
    one_minus_s = 1.0 - s
    top = (n + 1.0) ** one_minus_s
    return ((1.0 + u * (top - 1.0)) ** (1.0 / one_minus_s)) - 1.0


def _permute_rows(rank, rows):
    """Fixed bijection rank -> row so the hot rows are spread over the table."""
    mult = 2654435761
    while math.gcd(mult, rows) != 1:
        mult += 2
    return (rank * mult) % rows


def make_request(cfg, seed, tables=None, device=None):
    """One batch: dense [B, dense_in] fp32 ~N(0,1); per table lengths int32 [B] (power-law with
    exponent zipf_s on [1, max_len], rescaled to mean_len) and indices int64 (power-law over the
    rows through a fixed permutation).  Returned as torch tensors on `device` (CPU if None)."""
    tables = list(range(cfg.tables)) if tables is None else list(tables)
    g = torch.Generator(device="cpu").manual_seed(cfg.seed * 31 + seed)
    B = cfg.batch
    dense = torch.randn((B, cfg.dense_in), generator=g)
    ks = torch.arange(1, cfg.max_len + 1, dtype=torch.float64)
    pk = ks ** (-cfg.zipf_s)
    mean_raw = float((ks * pk).sum() / pk.sum())
    lengths, indices = {}, {}
    for t in tables:
        gt = torch.Generator(device="cpu").manual_seed((cfg.seed * 31 + seed) * 1009 + t)
        raw = _zipf_rank(torch.rand(B, generator=gt, dtype=torch.float64), cfg.max_len, cfg.zipf_s) + 1.0
        ln = torch.clamp(torch.round(raw * (cfg.mean_len / mean_raw)), 0, cfg.max_len).to(torch.int32)
        n = int(ln.sum())
        rank = torch.floor(_zipf_rank(torch.rand(n, generator=gt, dtype=torch.float64), cfg.rows, cfg.zipf_s))
        rank = torch.clamp(rank.to(torch.int64), 0, cfg.rows - 1)
        lengths[t], indices[t] = ln, _permute_rows(rank, cfg.rows)
    if device is not None:
        dense = dense.to(device)
        lengths = {t: v.to(device) for t, v in lengths.items()}
        indices = {t: v.to(device) for t, v in indices.items()}
    return dense, lengths, indices


def make_table(cfg, t, device):
    """Fused-rowwise uint8 table [rows, dim+8]: payload U{0..255}, scale U(0.001,0.01), offset U(-1,1)."""
    g = torch.Generator(device=device).manual_seed(cfg.seed * 7 + t)
    tab = torch.randint(0, 256, (cfg.rows, cfg.dim + 8), dtype=torch.uint8, device=device, generator=g)
    sc = torch.empty(cfg.rows, device=device).uniform_(0.001, 0.01, generator=g)
    of = torch.empty(cfg.rows, device=device).uniform_(-1, 1, generator=g)
    tab[:, cfg.dim:cfg.dim + 4] = sc.view(torch.uint8).view(cfg.rows, 4)
    tab[:, cfg.dim + 4:] = of.view(torch.uint8).view(cfg.rows, 4)
    return tab


# ------------------------------------------------------------------------------------------
# model parameters: float weights -> quantized constants, as Glow's graph creators do on the host
# ------------------------------------------------------------------------------------------
@dataclass
class QuantFC:
    """One RowwiseQuantizedFullyConnected (+ optional fused Relu) with its constants (numpy)."""
    w: np.ndarray            # int8 [N, K]
    w_scales: np.ndarray     # fp32 [N]
    w_offsets: np.ndarray    # int32 [N]
    bias: np.ndarray         # int32 [N]
    bias_scale: float
    in_scale: float
    in_offset: int
    out_scale: float
    out_offset: int
    relu: bool
    params: list = field(default_factory=list)  # six int32 [N] arrays


def he_normal(rng, fan_in, fan_out):
    return (rng.standard_normal((fan_out, fan_in)) * math.sqrt(2.0 / fan_in)).astype(np.float32)


def float_model(cfg):
    """He-normal fp32 weights [N, K] and small biases for the two MLPs."""
    rng = np.random.default_rng(cfg.seed + 17)
    layers = {"bottom": [], "top": []}
    k = cfg.dense_in
    for n in cfg.bottom:
        layers["bottom"].append((he_normal(rng, k, n), (rng.standard_normal(n) * 0.05).astype(np.float32)))
        k = n
    k = cfg.interaction_width
    for n in cfg.top:
        layers["top"].append((he_normal(rng, k, n), (rng.standard_normal(n) * 0.05).astype(np.float32)))
        k = n
    return layers


def float_forward(cfg, fm, dense, pooled):
    """fp32 forward of the dense part (torch, any device) recording (min, max) of every tensor that
    gets a quantized type: the calibration pass Glow runs in profiling mode."""
    ranges = {}
    rec = lambda name, x: ranges.__setitem__(name, (float(x.min()), float(x.max())))
    x = dense
    rec("dense", x)
    for i, (w, b) in enumerate(fm["bottom"]):
        x = torch.relu(x @ torch.as_tensor(w, device=x.device).T + torch.as_tensor(b, device=x.device))
        rec("bottom%d" % i, x)
    B, D = x.shape
    vecs = torch.cat([x[:, None, :], pooled.reshape(B, -1, D)], dim=1)
    z = vecs @ vecs.transpose(1, 2)
    ii, jj = torch.tril_indices(vecs.shape[1], vecs.shape[1], offset=-1)
    y = torch.cat([x, z[:, ii, jj]], dim=1)
    rec("interaction", y)
    for i, (w, b) in enumerate(fm["top"]):
        y = y @ torch.as_tensor(w, device=y.device).T + torch.as_tensor(b, device=y.device)
        if i + 1 < len(fm["top"]):
            y = torch.relu(y)
        rec("top%d" % i, y)
    return y, ranges


def quantize_model(cfg, fm, ranges):
    """Quantized constants for every FC: rowwise int8 weights (cfg.weights_schema), int32 bias with scale
    in_scale * (per-tensor weight scale), activation types from the calibrated ranges."""
    def tqp(name):
        return ops.choose_quantization_params(*ranges[name], ops.ASYMMETRIC)

    w_schema = ops.SYMMETRIC if cfg.weights_schema == "symmetric" else ops.ASYMMETRIC

    out = {"bottom": [], "top": []}
    prev = tqp("dense")
    out["dense_tqp"] = prev
    for part, first_in in (("bottom", "dense"), ("top", "interaction")):
        prev = tqp(first_in)
        for i, (w, b) in enumerate(fm[part]):
            q, sc, off = ops.tensor_rowwise_quantize_i8(w, w_schema)
            w_tensor_scale, _ = ops.choose_quantization_params(float(w.min()), float(w.max()), w_schema)
            bias_scale = float(np.float32(prev[0]) * np.float32(w_tensor_scale))
            o = tqp("%s%d" % (part, i))
            relu = not (part == "top" and i + 1 == len(fm[part]))
            fc = QuantFC(q, sc, off, ops.quantize_bias_i32(b, bias_scale, 0), bias_scale, prev[0], prev[1], o[0], o[1], relu)
            fc.params = ops.rowwise_requant_params(sc, prev[0], np.float32(bias_scale), o[0])
            out[part].append(fc)
            prev = o
    out["interaction_tqp"] = tqp("interaction")
    return out


class DeviceFC:
    """A QuantFC uploaded to one GPU."""

    def __init__(self, fc, device):
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        self.fc = fc
        self.w, self.bias, self.w_off = to(fc.w), to(fc.bias), to(fc.w_offsets)
        self.params = [to(a) for a in fc.params]
        self.row_sums = ops.i8_row_sums(self.w)
        self.flags = (ops.FC_FUSE_RELU if fc.relu else 0) | (ops.FC_WEIGHT_OFFSETS_ZERO if not fc.w_offsets.any() else 0)

    def __call__(self, x, out, workspace, status=None):
        return ops.rowwise_quantized_fc(x, self.w, self.bias, self.w_off, self.params[:3], self.params[3:],
                                        self.fc.out_offset, self.fc.in_offset, 0, weights_row_sums=self.row_sums,
                                        flags=self.flags, out=out, workspace=workspace, status=status)


# ------------------------------------------------------------------------------------------
# sharding plan (pure host logic; also exercised on CPU with gloo)
# ------------------------------------------------------------------------------------------
def tables_of_rank(cfg, rank, world):
    """Table-wise sharding: rank r owns tables {t : t % world == r}."""
    return [t for t in range(cfg.tables) if t % world == rank]


def batch_slice(cfg, rank, world):
    per = cfg.batch // world
    return rank * per, (rank + 1) * per


def exchange_all_to_all(pooled_by_dest, cfg, rank, world, group=None):
    """The exchange as one torch.distributed.all_to_all_single.
    pooled_by_dest: [world, B/world, T_local, D] (this rank's tables, bags grouped by destination).
    Returns [B/world, T, D] for this rank's batch slice, tables in global order."""
    import torch.distributed as dist
    per = cfg.batch // world
    counts = [len(tables_of_rank(cfg, r, world)) for r in range(world)]
    D = pooled_by_dest.shape[-1]
    recv = torch.empty((sum(counts) * per * D,), dtype=pooled_by_dest.dtype, device=pooled_by_dest.device)
    send = pooled_by_dest.reshape(-1)
    t_local = counts[rank]
    dist.all_to_all_single(recv, send, output_split_sizes=[c * per * D for c in counts],
                           input_split_sizes=[t_local * per * D] * world, group=group)
    out = torch.empty((per, cfg.tables, D), dtype=pooled_by_dest.dtype, device=pooled_by_dest.device)
    pos = 0
    for r in range(world):
        tabs = tables_of_rank(cfg, r, world)
        if tabs:
            out[:, tabs, :] = recv[pos:pos + len(tabs) * per * D].view(per, len(tabs), D)
        pos += len(tabs) * per * D
    return out


# ------------------------------------------------------------------------------------------
# one rank of the model
# ------------------------------------------------------------------------------------------
class DLRMRank:
    """The part of the model one GPU runs: its tables for the whole batch, the dense layers for
    its slice of the batch.  exchange: "local" (world 1), "nccl", "fused", or "emulated" (several
    ranks living in one process on one GPU, for tests: peers are wired with set_peers)."""

    def __init__(self, cfg, qm, tables, rank=0, world=1, device="cuda", exchange="local", group=None, rendezvous="flags"):
        self.cfg, self.rank, self.world, self.device = cfg, rank, world, torch.device(device)
        self.exchange, self.group = exchange, group
        self.my_tables = tables_of_rank(cfg, rank, world)
        self.tables = tables  # dict table id -> uint8 [rows, dim+8] on this device
        self.per = cfg.batch // world
        self.bottom = [DeviceFC(fc, self.device) for fc in qm["bottom"]]
        self.top = [DeviceFC(fc, self.device) for fc in qm["top"]]
        self.dense_tqp, self.inter_tqp = qm["dense_tqp"], qm["interaction_tqp"]
        self.status = ops.new_status(self.device)
        dev, per, D, T = self.device, self.per, cfg.dim, cfg.tables
        widths = [cfg.dense_in] + list(cfg.bottom)
        self.act_b = [torch.empty((per, w), dtype=torch.int8, device=dev) for w in widths]
        widths = [cfg.interaction_width] + list(cfg.top)
        self.act_t = [torch.empty((per, w), dtype=torch.int8, device=dev) for w in widths]
        self.x0 = torch.empty((per, D), dtype=torch.float32, device=dev)
        self.result = torch.empty((per, 1), dtype=torch.float32, device=dev)
        need = max(ops.i8_gemm_workspace_bytes(per, k, n) for k, n in
                   zip([cfg.dense_in] + list(cfg.bottom) + [cfg.interaction_width] + list(cfg.top),
                       list(cfg.bottom) + [0] + list(cfg.top)) if n)
        self.ws = torch.empty(need, dtype=torch.uint8, device=dev)
        # the bottom MLP does not depend on the pooled vectors: it runs on a stream of its own,
        # beside the pooling kernel, with a workspace of its own
        self.ws_bottom = torch.empty(need, dtype=torch.uint8, device=dev)
        self.side = torch.cuda.Stream(device=dev)
        self.ones = None
        # receive slabs [per, T, D] (two, alternating by step) and, for "nccl", the send buffer
        self.step = 0
        self.peers = None
        self.token = torch.zeros(1, dtype=torch.float32, device=dev)
        if exchange == "fused":
            self.slab_buf = [ops.PeerBuffer(per * T * D * 4) for _ in range(2)]
            self.slabs = [b.as_tensor((per, T, D), torch.float32) for b in self.slab_buf]
            # the ranks' rendezvous: a flag per peer plus this rank's step count, written by a small
            # kernel of the library (ops.peer_rendezvous); "nccl" keeps a one-element all-reduce instead
            self.rendezvous = rendezvous
            self.flag_buf = ops.PeerBuffer(8 * (world + 1))
            self.flag_buf.as_tensor((8 * (world + 1),), torch.uint8).zero_()
            self.flag_peers = None
        else:
            self.slabs = [torch.empty((per, T, D), dtype=torch.float32, device=dev) for _ in range(2)]
        if exchange == "nccl":
            # send: bags grouped by destination rank; recv: one [per, T_r, D] block from every rank
            self.send = torch.empty((world, per, len(self.my_tables), D), dtype=torch.float32, device=dev)
            self.recv = torch.empty((per * T * D,), dtype=torch.float32, device=dev)

    def connect_peers(self):
        """fused exchange: swap IPC handles of the receive slabs with every rank."""
        import torch.distributed as dist
        handles = [None] * self.world
        dist.all_gather_object(handles, [b.handle for b in self.slab_buf] + [self.flag_buf.handle], group=self.group)
        self.peers = []  # [slab][rank] -> base address
        for s in range(2):
            self.peers.append([self.slab_buf[s].ptr if r == self.rank else self.slab_buf[s].open(handles[r][s])
                               for r in range(self.world)])
        flags = [self.flag_buf.ptr if r == self.rank else self.flag_buf.open(handles[r][2]) for r in range(self.world)]
        self.flag_peers = torch.tensor(flags, dtype=torch.int64).to(self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # every rank's flags are zeroed and mapped before the first rendezvous

    def set_peers(self, ranks):
        """emulated exchange: every rank's slabs are plain tensors of this process."""
        self.peers = [[r.slabs[s].data_ptr() for r in ranks] for s in range(2)]

    def release(self):
        if self.exchange == "fused":
            for b in self.slab_buf + [self.flag_buf]:
                b.release()

    # -- sparse part ---------------------------------------------------------------------
    def prepare(self, lengths, indices, slab):
        """Binds one request (lengths/indices: dicts over MY tables, whole batch, on this device)
        to the receive slab `slab` (0/1).  Returns the bound launch; binding is host work plus one
        small descriptor upload, so a serving loop does it once per request buffer."""
        D, T = self.cfg.dim, self.cfg.tables
        n_max = max([int(indices[t].shape[0]) for t in self.my_tables] + [1])
        if self.ones is None or self.ones.shape[0] < n_max:
            self.ones = torch.ones(n_max, dtype=torch.float32, device=self.device)
        tabs = [self.tables[t] for t in self.my_tables]
        w = [self.ones[:indices[t].shape[0]] for t in self.my_tables]
        idx = [indices[t] for t in self.my_tables]
        ln = [lengths[t] for t in self.my_tables]
        b = ops.SlwsBatch(ops.UINT8_FUSED, D + 8, torch.int64, device=self.device)
        if self.exchange == "nccl":
            # bags grouped by destination rank: send[r, b, j, :] -- one scatter target per rank
            base, tl = self.send.data_ptr(), len(self.my_tables)
            scatter = [[base + ((r * self.per * tl) + j) * D * 4 for r in range(self.world)] for j in range(tl)]
            b.bind(tabs, w, idx, ln, None, dest_stride=tl * D, scatter=scatter, bags_per_dest=self.per)
        else:
            bases = self.peers[slab] if self.exchange in ("fused", "emulated") else [self.slabs[slab].data_ptr()]
            scatter = [[bases[r] + t * D * 4 for r in range(self.world)] for t in self.my_tables]
            b.bind(tabs, w, idx, ln, None, dest_stride=T * D, scatter=scatter, bags_per_dest=self.per)
        return b

    def pool_and_exchange(self, bound, slab):
        import torch.distributed as dist
        bound.run(self.status)
        if self.exchange == "nccl":
            T, D, tl = self.cfg.tables, self.cfg.dim, len(self.my_tables)
            if T % self.world == 0:
                # every buffer exists already and nothing below touches the host, so the step can be
                # captured in a CUDA graph like the fused form: equal blocks out, equal blocks in,
                # then one strided copy puts table j of rank r at column j * world + r
                dist.all_to_all_single(self.recv, self.send.view(-1), group=self.group)
                self.slabs[slab].view(self.per, tl, self.world, D).copy_(
                    self.recv.view(self.world, self.per, tl, D).permute(1, 2, 0, 3))
            else:
                self.slabs[slab].copy_(exchange_all_to_all(self.send, self.cfg, self.rank, self.world, self.group))
        elif self.exchange == "fused":
            # every rank's stores into every slab are complete once all pooling kernels have
            # finished: the rendezvous is a kernel on the stream (it never blocks the host and can
            # be captured in a CUDA graph, unlike a barrier)
            if self.rendezvous == "flags":
                ops.peer_rendezvous(self.flag_buf.ptr, self.flag_peers, self.world, self.rank, self.status)
            else:
                dist.all_reduce(self.token, group=self.group)
        return self.slabs[slab]

    # -- dense part ----------------------------------------------------------------------
    def bottom_forward(self, dense_slice):
        ops.element_quantize_i8(dense_slice, self.dense_tqp[0], self.dense_tqp[1], out=self.act_b[0])
        for i, fc in enumerate(self.bottom):
            fc(self.act_b[i], self.act_b[i + 1], self.ws_bottom, self.status)
        last = self.bottom[-1].fc
        ops.element_dequantize_i8(self.act_b[-1], last.out_scale, last.out_offset, out=self.x0)
        return self.x0

    def dense_forward(self, dense_slice, pooled):
        self.bottom_forward(dense_slice)
        return self.top_forward(pooled)

    def top_forward(self, pooled):
        ops.pairwise_dot_interaction(self.x0, pooled, quant=self.inter_tqp, out=self.act_t[0])
        for i, fc in enumerate(self.top):
            fc(self.act_t[i], self.act_t[i + 1], self.ws, self.status)
        last = self.top[-1].fc
        ops.element_dequantize_i8(self.act_t[-1], last.out_scale, last.out_offset, out=self.result)
        return self.result

    def forward(self, dense_slice, bound_pair):
        """One step: bound_pair[slab] is the request bound to each of the two receive slabs."""
        slab = self.step & 1
        main = torch.cuda.current_stream(self.device)
        self.side.wait_stream(main)          # the dense features (and the last step's x0 readers) are ready
        # (ordinary launches on the side stream: a contraction waiting for its predecessor there would
        # hold an SM's shared memory that the pooling kernel on the main stream can use)
        with torch.cuda.stream(self.side), ops.programmatic_launch(False):
            self.bottom_forward(dense_slice)
        pooled = self.pool_and_exchange(bound_pair[slab], slab)
        main.wait_stream(self.side)
        out = self.top_forward(pooled)
        self.step += 1
        return out

    def forward_request(self, dense_slice, lengths, indices):
        slab = self.step & 1
        pair = [None, None]
        pair[slab] = self.prepare(lengths, indices, slab)
        return self.forward(dense_slice, pair)

    @property
    def launches_per_step(self):
        # segments + gather, quantize, FCs, dequantize x2, interaction
        return 2 + 1 + len(self.bottom) + 1 + 1 + len(self.top) + 1


def fixed_ranges(cfg):
    """Activation ranges of about the calibrated size, for runs that only time one rank's share
    of a partitioned model and cannot calibrate (no pooled vectors of the other ranks)."""
    r = {"dense": (-4.5, 4.5), "interaction": (-60.0, 60.0)}
    for i in range(len(cfg.bottom)):
        r["bottom%d" % i] = (0.0, 6.0)
    for i in range(len(cfg.top)):
        r["top%d" % i] = (0.0, 30.0) if i + 1 < len(cfg.top) else (-30.0, 30.0)
    return r


def calibrate(cfg, fm, tables, device, rank=0, world=1, group=None):
    """Calibration pass: one seeded batch through the fp32 model (pooling in fp32 torch).
    `tables` holds this rank's tables; with world > 1 the pooled vectors of the calibration batch
    are all-gathered so every rank derives the same ranges."""
    mine = tables_of_rank(cfg, rank, world)
    dense, lengths, indices = make_request(cfg, 999_983, tables=mine, device=device)
    D = cfg.dim
    local = torch.empty((cfg.batch, len(mine), D), dtype=torch.float32, device=device)
    for j, t in enumerate(mine):
        tab = tables[t]
        rows = tab[indices[t]]
        sc = rows[:, D:D + 4].contiguous().view(torch.float32)
        of = rows[:, D + 4:].contiguous().view(torch.float32)
        deq = rows[:, :D].float() * sc + of
        seg = torch.repeat_interleave(torch.arange(cfg.batch, device=device), lengths[t].long())
        local[:, j].zero_().index_add_(0, seg, deq)
    pooled = torch.empty((cfg.batch, cfg.tables, D), dtype=torch.float32, device=device)
    if world == 1:
        pooled[:, mine] = local
    else:
        import torch.distributed as dist
        for r in range(world):
            tabs = tables_of_rank(cfg, r, world)
            buf = local if r == rank else torch.empty((cfg.batch, len(tabs), D), dtype=torch.float32, device=device)
            dist.broadcast(buf, src=r, group=group)
            pooled[:, tabs] = buf
    _, ranges = float_forward(cfg, fm, dense, pooled)
    return ranges
