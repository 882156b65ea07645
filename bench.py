#!/usr/bin/env python
"""Benchmark of the embedding gather-pool hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("step" = one pooled lookup of one batch over all tables of a rank):
FusedRowwiseQuantizedSparseLengthsWeightedSum with the first benchmark configuration's table
and bag law -- 1,000,000 x 64 uint8 rows fused with fp32 scale/offset (72 B per row), 1024
bags per table, lengths clamp(Poisson(32),1,128), int64 indices uniform over the rows, fp32
weights U(0,1) -- over T distinct tables in ONE launch (the reference's SLS benchmark does the
same with numSLSNodes, tests/benchmark/SLSBench.cpp:49-104).  One table alone moves 3 MB per
launch out of an L2-resident 72 MB table, which measures launch latency, not HBM; T tables
(18 GB, far beyond the 126 MB L2) make it a bandwidth measurement.  At N > 1 every rank owns
T tables of its own (table-wise sharding, no data-path collective): weak scaling.

metric: algorithmic GB/s = [sum(lengths) * (72 + 8 + 4) + bags * (4 + 256)] / time.
Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, DIM, BATCH = 1_000_000, 64, 1024
IN_LINE = DIM + 8
# DRAM bytes per gathered 72-byte row of the uint8 gather kernel: dram__bytes_read.sum +
# dram__bytes_write.sum of one launch over 64 tables (4.6 waves of blocks, 2.10 M rows), from the
# ncu capture summarised in profiles/.  ncu cannot run inside the timed region, so `traffic` is
# this figure x the rows of the timed launch (traffic is proportional to rows: every row is
# fetched once, L2 hit rate 13 %).
NCU_DRAM_BYTES_PER_ROW = 205.6
METRIC = "frwq_slws_hbm_gbps"
UNIT = "GB/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tables", type=int, default=256, help="tables per GPU (T)")
    ap.add_argument("--requests", type=int, default=4, help="distinct pre-generated batches rotated over the steps")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="slws", choices=["slws", "int8_fc", "slws4", "dlrm", "resnet50", "tbe", "dyn_fc"],
                    help="slws: the headline gather-pool line (default); int8_fc: the rowwise int8 FC line; "
                         "slws4: the 4-bit fused-rowwise sweep point selected by --dim; dlrm / resnet50: the "
                         "recommendation model / the int8 ResNet-50 alone (the default line carries both as extras); "
                         "tbe: table-batched embedding bags (IntNBitSplitEmbeddingBags) over tables of --tbe-type; "
                         "dyn_fc: DynamicRowwiseQuantizedFullyConnected at the shape of the int8 FC line")
    ap.add_argument("--tbe-type", default="int4", choices=["fp16", "int8", "int4"], help="tbe: element type of the tables")
    ap.add_argument("--tbe-out", default="fp16", choices=["fp16", "fp32"], help="tbe: element type of the result")
    ap.add_argument("--dim", type=int, default=128, help="slws4: embedding width (32, 64, 128 or 256)")
    ap.add_argument("--table-gb", type=float, default=40.0, help="slws4: total table bytes per GPU, in GB")
    ap.add_argument("--row-bytes", type=int, default=0,
                    help="slws: store the tables with rows padded to this many bytes (0: the dense 72-byte rows)")
    ap.add_argument("--shard", default="tables", choices=["tables", "rows", "rows-routed"],
                    help="slws4 at N > 1: every rank owns whole tables (no exchange); row ranges of every table, every "
                         "rank filtering the whole request; or row ranges with the request routed to the owning rank "
                         "beforehand (each rank is handed only the indices of its rows)")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary int8 FC measurement")
    ap.add_argument("--as-rank-of", type=int, default=0,
                    help="dlrm on ONE GPU: run only what rank 0 of an N-way table partition runs in a step (its "
                         "tables for the whole batch, the dense layers for a 1/N slice of the batch; the exchange "
                         "stores go to its own slab) -- the per-rank launch list of an N-GPU step, for profiling")
    return ap.parse_args()


def measured_peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def algorithmic_bytes(num_indices, bags):
    return num_indices * (IN_LINE + 8 + 4) + bags * (4 + DIM * 4)


def request_host(tables, seed):
    """One batch for `tables` tables: lengths [T, B], and per-table indices / weights."""
    rng = np.random.Generator(np.random.PCG64(seed))
    lengths = np.clip(rng.poisson(32, (tables, BATCH)), 1, 128).astype(np.int32)
    n = lengths.sum(1)
    total = int(n.sum())
    indices = rng.integers(0, ROWS, total, dtype=np.int64)
    weights = rng.random(total, dtype=np.float32)
    starts = np.concatenate([[0], np.cumsum(n)]).astype(np.int64)
    return lengths, indices, weights, starts


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


class HostPipeline:
    """The end-to-end legs keep two requests in flight, as a serving loop does: while request i
    runs, the inputs of request i+1 are copied in and the result of request i-1 is copied out, on
    three streams ordered by events.  Buffer set b (staging inputs, result) is reused by every
    NBUF-th request; every step's copies stay inside the timed region."""

    def __init__(self, torch, nbuf=2):
        self.torch, self.nbuf = torch, nbuf
        self.s_in, self.s_run, self.s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        self.ev_in = [torch.cuda.Event() for _ in range(nbuf)]
        self.ev_run = [torch.cuda.Event() for _ in range(nbuf)]
        self.ev_out = [torch.cuda.Event() for _ in range(nbuf)]
        for st in (self.s_in, self.s_run, self.s_out):
            st.wait_stream(torch.cuda.current_stream())

    def step(self, b, copy_in, run, copy_out):
        torch = self.torch
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.ev_run[b])    # the kernels that last read this staging set are done
            copy_in()
            self.ev_in[b].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[b])
            self.s_run.wait_event(self.ev_out[b])   # the result buffer has been copied out
            run()
            self.ev_run[b].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[b])
            copy_out()
            self.ev_out[b].record(self.s_out)

    def timed(self, fn, n):
        """fn(i) enqueues step i through `step`; -> milliseconds from the first copy-in to the last copy-out."""
        torch = self.torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(self.s_in)
        for i in range(n):
            fn(i)
        e1.record(self.s_out)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)


def cpu_reference_rate(tables_host, seconds, threads, distinct=24):
    """Times the reference's own kernel (libjit, fast-math build as Glow ships it; the plain-C
    port when that build is absent) on host threads, one table per call, tables spread over the
    threads the way Glow runs one CPU device per core.  Every pass pools a different batch
    (`distinct` pre-generated batches, cycled) so the rows it gathers are not cache-resident
    from the pass before.  -> (GB/s, kind, passes, seconds)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as orc
    if orc.ref_available("fast"):
        ref = orc.LibjitRef("fast")
        fn, kind = ref.frwq_slws, "reference"
    else:
        orc.lib()
        fn, kind = (lambda t, w, i, l: orc.frwq_slws_u8_f32(t, w, i, l)), "port"
    S = len(tables_host)
    reqs = [request_host(S, 5000 + i) for i in range(distinct)]

    def one(args):
        k, (lengths, indices, weights, starts) = args
        a, b = starts[k], starts[k + 1]
        fn(tables_host[k], weights[a:b], indices[a:b], lengths[k])

    moved = 0
    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(one, [(k, reqs[0]) for k in range(S)]))  # warm-up pass
        passes, t0 = 0, time.perf_counter()
        while True:
            rq = reqs[(passes + 1) % distinct]
            list(ex.map(one, [(k, rq) for k in range(S)]))
            moved += algorithmic_bytes(int(rq[3][S]), S * BATCH)
            passes += 1
            dt = time.perf_counter() - t0
            if dt >= seconds:
                break
    return moved / dt / 1e9, kind, passes, dt


def make_table_host(seed):
    from glow_b200 import workloads
    return workloads.fused_table_u8(ROWS, DIM, seed, 0)


def run_reference(args):
    """--impl reference: the reference's CPU kernel on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    S = min(args.tables, max(threads, 16))
    tables = [make_table_host(1000 + k) for k in range(S)]
    per_step = max(0.5, min(4.0, 60.0 / max(1, args.steps + args.warmup)))
    vals = []
    kind = "port"
    for i in range(args.warmup + args.steps):
        v, kind, passes, dt = cpu_reference_rate(tables, per_step, threads)
        if i >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals)) if vals else 0.0
    nbytes = algorithmic_bytes(int(S * BATCH * 32.0), S * BATCH)
    sample = ("%d of %d tables per pass, a different batch each pass, passes repeated for %.1f s per step"
              % (S, args.tables, per_step))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": nbytes / (value * 1e9) * 1e3 if value else None,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.tables),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def measured_peak_int8(ops=None):
    """The int8 ceiling, measured in this run: the tensor pipe issuing 128 x 256 x 32 int8 MMAs
    back to back on resident tiles, one CTA per SM, nothing loaded or stored (the driver's file of
    measured peaks has bf16 only).  -> (TOP/s, how)."""
    if ops is not None:
        try:
            return float(ops.i8_mma_issue_rate()), "measured here: tcgen05 kind::i8 issue loop on resident tiles, all SMs"
        except Exception as ex:  # noqa: BLE001
            print("int8 ceiling probe failed: %r" % (ex,), file=sys.stderr)
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return 2.0 * float(json.load(open(p))["bf16_tflops"]), "2 x measured bf16 burst (the probe did not run)"
        except Exception:
            pass
    return 2.0 * 1590.0, "2 x fallback bf16 (the probe did not run)"


FC_M, FC_K, FC_N = 2048, 4096, 4096


def int8_fc_measure(torch, ops, dev, steps, warmup, seed=0):
    """RowwiseQuantizedFullyConnected M2048 K4096 N4096 (second benchmark configuration):
    device-resident TOPS, end-to-end TOPS (activations in from pinned host memory, int8 result
    out), and the library int8 GEMM (torch._int_mm -> cuBLASLt, int32 result, no requantisation)
    on the same operands for context.  Weight row sums are precomputed once, as a backend does
    at network-load time."""
    from glow_b200 import workloads
    c = workloads.config2(M=FC_M, K=FC_K, N=FC_N, seed=workloads.MASTER_SEED + seed)
    params = ops.rowwise_requant_params(c["w_scales"], c["in_scale"], c["bias_scale"], c["out_scale"])
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    p = [to(a) for a in params]
    w, bias, wo = to(c["w"]), to(c["bias"]), to(c["w_offsets"])
    rs = ops.i8_row_sums(w)
    # activations: several distinct batches so consecutive steps do not re-read an L2-resident input
    host_in = [torch.from_numpy(np.random.default_rng(seed + i).integers(-128, 128, (FC_M, FC_K), dtype=np.int8)).pin_memory()
               for i in range(4)]
    dev_in = [h.to(dev) for h in host_in]
    out = torch.empty((FC_M, FC_N), dtype=torch.int8, device=dev)
    out_host = torch.empty((FC_M, FC_N), dtype=torch.int8).pin_memory()
    stage = torch.empty((FC_M, FC_K), dtype=torch.int8, device=dev)
    ws = torch.empty(ops.i8_gemm_workspace_bytes(FC_M, FC_K, FC_N), dtype=torch.uint8, device=dev)
    status = ops.new_status(dev)

    def run(x):
        ops.rowwise_quantized_fc(x, w, bias, wo, p[:3], p[3:], c["out_offset"], c["in_offset"], c["bias_offset"],
                                 weights_row_sums=rs, flags=ops.FC_WEIGHT_OFFSETS_ZERO, out=out, workspace=ws,
                                 status=status)

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    for i in range(max(3, warmup)):
        run(dev_in[i % 4])
    ms = timed(lambda i: run(dev_in[i % 4]), steps)

    pipe = HostPipeline(torch, 2)
    stages = [stage, torch.empty_like(stage)]
    outs = [torch.empty_like(out), torch.empty_like(out)]
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]

    def run_into(x, o):
        ops.rowwise_quantized_fc(x, w, bias, wo, p[:3], p[3:], c["out_offset"], c["in_offset"], c["bias_offset"],
                                 weights_row_sums=rs, flags=ops.FC_WEIGHT_OFFSETS_ZERO, out=o, workspace=ws,
                                 status=status)

    def e2e(i):
        b = i % 2
        pipe.step(b, lambda: stages[b].copy_(host_in[i % 4], non_blocking=True), lambda: run_into(stages[b], outs[b]),
                  lambda: out_hosts[b].copy_(outs[b], non_blocking=True))

    for i in range(4):
        e2e(i)
    e2e_steps = max(4, min(steps, 20))
    e2e_ms = pipe.timed(e2e, e2e_steps) / e2e_steps
    assert int(status.item()) == 0
    ops_per_step = 2.0 * FC_M * FC_N * FC_K
    lib_tops = None
    try:
        wt = w.t()
        for i in range(3):
            torch._int_mm(dev_in[i % 4], wt)
        lib_ms = timed(lambda i: torch._int_mm(dev_in[i % 4], wt), steps)
        lib_tops = ops_per_step / (lib_ms * 1e-3) / 1e12
    except Exception:
        pass
    return {"ms": ms, "tops": ops_per_step / (ms * 1e-3) / 1e12, "e2e_ms": e2e_ms,
            "e2e_tops": ops_per_step / (e2e_ms * 1e-3) / 1e12, "e2e_steps": e2e_steps,
            "h2d": FC_M * FC_K, "d2h": FC_M * FC_N, "library_int8_gemm_tops": lib_tops, "ops": ops_per_step}


def int8_fc_cpu_rate(seconds, threads):
    """The reference's libjit_rowwise_quantized_fc_i8_i32 (fast-math build; the plain-C port when that
    build is absent) on a slice of the batch rows of the same layer: 8 rows per host thread per call,
    repeated for `seconds`.  The kernel's cost is linear in the rows, so TOP/s of the slice is
    TOP/s of the layer.  -> (TOP/s, kind, sample description)."""
    from oracle import oracle as orc
    from glow_b200 import workloads
    c = workloads.config2(M=FC_M, K=FC_K, N=FC_N)
    pre = orc.rowwise_requant_params(c["w_scales"], c["in_scale"], c["bias_scale"], c["out_scale"])
    if orc.ref_available("fast"):
        fn, kind = orc.LibjitRef("fast").rowwise_quantized_fc_i8_i32, "reference"
    else:
        fn, kind = orc.rowwise_quantized_fc_i8_i32, "port"
    rows = 8 * threads
    x = np.ascontiguousarray(c["inp"][:rows])
    call = lambda: fn(x, c["w"], c["bias"], c["w_offsets"], pre[:3], pre[3:], c["out_offset"], c["in_offset"],
                      c["bias_offset"], threads=threads)
    call()
    n, t0 = 0, time.perf_counter()
    while True:
        call()
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    tops = n * 2.0 * rows * FC_N * FC_K / dt / 1e12
    return tops, kind, "%d of %d batch rows per call (8 per thread, %d host threads), %d calls in %.1f s" % (
        rows, FC_M, threads, n, dt)


def fc_config():
    return {"workload": "RowwiseQuantizedFullyConnected int8: M=2048 K=4096 N=4096, activations U[-128,127] "
                        "(scale 0.05, offset 3), weights U[-127,127] with per-row scales U(0.001,0.02) and zero "
                        "offsets, int32 bias U[-2^16,2^16] (scale 5e-4), int8 result (scale 0.5, offset 0), "
                        "integer requantisation fused in the epilogue; weight row sums precomputed",
            "M": FC_M, "K": FC_K, "N": FC_N,
            "l2_policy": "four distinct activation batches rotated; weights (16 MB) stay L2-resident as in serving"}


def run_int8_fc_line(args):
    """--workload int8_fc: the dense line.  At N > 1 every rank runs its own batch (batch-sharded
    replicas, no collective): weak scaling."""
    import torch
    import torch.distributed as dist
    from glow_b200 import ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    r = int8_fc_measure(torch, ops, dev, args.steps, args.warmup, seed=rank)
    t_end = time.time() + 1.0
    while len(sampler.lines) < 8 and time.time() < t_end:
        time.sleep(0.05)
    clocks = sampler.stop()
    times = torch.tensor([r["ms"], r["e2e_ms"]], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(times[0]), float(times[1])
    if rank == 0:
        peak, src = measured_peak_int8(ops)
        tops = world * r["ops"] / (ms * 1e-3) / 1e12
        line = {"metric": "int8_fc_tops", "value": tops, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "s8 x s8 -> s32", "data": "synthetic", "config": fc_config(),
                "roofline": {"bound": "tensor", "achieved": r["tops"], "peak": peak, "unit": "TOP/s",
                             "frac": r["tops"] / peak, "peak_source": src, "nominal_dense_int8_tops": 4500.0,
                             "frac_of_nominal": r["tops"] / 4500.0,
                             "library_int8_gemm_tops": r["library_int8_gemm_tops"],
                             # DRAM bytes per launch from the ncu capture in profiles/ (the 8 MB result stays in L2)
                             "traffic": 25.4e6,
                             "kernel": "i8_gemm_requant_kernel<240,4,0>", "launch_us": r["ms"] * 1e3},
                "e2e": {"value": world * r["ops"] / (e2e_ms * 1e-3) / 1e12, "unit": "TOP/s",
                        "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"], "steps": r["e2e_steps"],
                        "ms_per_step": e2e_ms},
                "gpu_launches": args.steps, "clocks": clocks}
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, kind, sample = int8_fc_cpu_rate(min(args.cpu_seconds, 10.0), threads)
            line["cpu_baseline"] = {"value": v, "unit": "TOP/s", "cores": threads, "kind": kind, "sample": sample}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def dlrm_partition_checks(torch, dist, dev, rank, world, cfg, qm, tables):
    """Result checks of the partitioned model on the real GPUs, before anything is timed
    (the reference requires a partitioned run to equal the unpartitioned one bit for bit,
    tests/unittests/RecommendationSystemTest.cpp:1155-1226):
      exchange_forms_agree   the fused peer-store exchange and the NCCL all-to-all give the same
                             pooled slabs and the same scores on every rank;
      matches_unpartitioned  the scores of all ranks, gathered, equal what rank 0 computes with
                             all tables on one GPU.
    Raises if either is false."""
    from glow_b200 import dlrm
    mine = dlrm.tables_of_rank(cfg, rank, world)
    lo, hi = dlrm.batch_slice(cfg, rank, world)
    dense, lengths, indices = dlrm.make_request(cfg, 4242, tables=mine, device=dev)
    got = {}
    for exchange in ("fused", "nccl"):
        model = dlrm.DLRMRank(cfg, qm, tables, rank, world, dev, exchange)
        if exchange == "fused":
            model.connect_peers()
        outs = []
        for _ in range(2):  # both receive slabs
            out = model.forward_request(dense[lo:hi].contiguous(), lengths, indices)
            torch.cuda.synchronize()
            dist.barrier()
            outs.append((out.clone(), model.slabs[(model.step - 1) & 1].clone()))
        assert int(model.status.item()) == 0
        got[exchange] = outs
        dist.barrier()
        model.release()
        del model
    same = all(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) for a, b in zip(got["fused"], got["nccl"]))
    same = same and torch.equal(got["fused"][0][0], got["fused"][1][0])
    gathered = [torch.empty_like(got["fused"][0][0]) for _ in range(world)]
    dist.all_gather(gathered, got["fused"][0][0])
    whole_ok = True
    if rank == 0:
        all_tables = {t: (tables[t] if t in tables else dlrm.make_table(cfg, t, dev)) for t in range(cfg.tables)}
        d1, l1, i1 = dlrm.make_request(cfg, 4242, device=dev)
        single = dlrm.DLRMRank(cfg, qm, all_tables, 0, 1, dev, "local")
        want = single.forward_request(d1, l1, i1)
        torch.cuda.synchronize()
        whole_ok = torch.equal(torch.cat(gathered, 0), want)
        del single, all_tables
        torch.cuda.empty_cache()
    flags = torch.tensor([int(same), int(whole_ok)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    res = {"exchange_forms_agree": bool(int(flags[0])), "matches_unpartitioned": bool(int(flags[1]))}
    if not (res["exchange_forms_agree"] and res["matches_unpartitioned"]):
        raise AssertionError("partitioned DLRM results differ: %r" % res)
    return res


def dlrm_measure(torch, dist, dev, rank, world, steps, warmup, exchanges, as_rank_of=0):
    """DLRM-style model of the fourth benchmark configuration: 64 tables x 4,000,000 rows x 128
    (uint8 fused rows), batch 4096, power-law bag lengths (mean 40, max 200) and row indices,
    bottom MLP 256-512-256-128, pairwise-dot interaction (2208 wide), top MLP 2208-1024-1024-512-1,
    all dense layers int8 rowwise FC.  Tables sharded by table over the ranks, dense layers
    batch-sharded; samples/s = 4096 / (time per step), device-timed, max over ranks.
    Returns {exchange: {...}} for every exchange form in `exchanges`."""
    from glow_b200 import dlrm
    cfg = dlrm.DLRMConfig()
    part = as_rank_of if (as_rank_of and world == 1) else world   # ways the model is partitioned
    mine = dlrm.tables_of_rank(cfg, rank, part)
    tables = {t: dlrm.make_table(cfg, t, dev) for t in mine}
    fm = dlrm.float_model(cfg)
    if part != world:
        ranges = dlrm.fixed_ranges(cfg)   # one rank alone cannot calibrate: timing only
    else:
        ranges = dlrm.calibrate(cfg, fm, tables, dev, rank, world)
    qm = dlrm.quantize_model(cfg, fm, ranges)
    lo, hi = dlrm.batch_slice(cfg, rank, part)
    checks = {}
    if world > 1:
        checks = dlrm_partition_checks(torch, dist, dev, rank, world, cfg, qm, tables)
    R = 2
    host = []
    for r in range(R):
        dense, lengths, indices = dlrm.make_request(cfg, 100 + r, tables=mine)
        host.append((dense[lo:hi].contiguous().pin_memory(), {t: v.pin_memory() for t, v in lengths.items()},
                     {t: v.pin_memory() for t, v in indices.items()}))
    results = {}
    for exchange in exchanges:
        form = exchange
        rendezvous = "flags"
        if exchange == "fused_nccl_rendezvous":  # the fused exchange with a one-element all-reduce as the rendezvous
            exchange, rendezvous = "fused", "nccl"
        model = dlrm.DLRMRank(cfg, qm, tables, rank, part, dev, exchange, rendezvous=rendezvous)
        if exchange == "fused":
            model.connect_peers()
        elif exchange == "emulated":
            model.set_peers([model] * part)
        devr = [(h[0].to(dev), {t: v.to(dev) for t, v in h[1].items()}, {t: v.to(dev) for t, v in h[2].items()})
                for h in host]
        bound = [[model.prepare(d[1], d[2], slab) for slab in range(2)] for d in devr]

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def step(i):
            return model.forward(devr[i % R][0], bound[i % R])

        for i in range(max(4, warmup)):
            step(i)
        barrier()
        # The step is a dozen short launches: replay it from a CUDA graph (two consecutive steps
        # per graph, one per receive slab) so the host's launch cost stays off the device's
        # critical path.  Falls back to eager launches if capture is not possible.
        graph, graphed = None, False
        if model.step % 2 == 0:
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                        step(0)
                        step(1)
                torch.cuda.current_stream().wait_stream(side)
                graphed = True
            except Exception as ex:  # noqa: BLE001
                graph, graphed = None, False
                torch.cuda.synchronize()
                if rank == 0:
                    print("dlrm: CUDA graph capture failed (%s); timing eager launches" % type(ex).__name__,
                          file=sys.stderr)
        agree = torch.tensor([1 if graphed else 0], device=dev)
        if world > 1:
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        graphed = bool(int(agree.item()))
        if graphed:
            for i in range(2):
                graph.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if graphed:
            for i in range((steps + 1) // 2):
                graph.replay()
            timed_steps = 2 * ((steps + 1) // 2)
        else:
            for i in range(steps):
                step(i)
            timed_steps = steps
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / timed_steps
        assert int(model.status.item()) == 0
        # end to end: this rank's slice of the dense features and the lookups of its tables come
        # from pinned host memory every step; the scores go back to the host
        stage = [(torch.empty_like(d[0]), {t: torch.empty_like(v) for t, v in d[1].items()},
                  {t: torch.empty_like(v) for t, v in d[2].items()}) for d in devr]
        ebound = [[model.prepare(sg[1], sg[2], slab) for slab in range(2)] for sg in stage]
        out_host = torch.empty((hi - lo, 1), dtype=torch.float32).pin_memory()
        h2d = sum(host[0][0].numel() * 4 + sum(v.numel() * 4 for v in host[0][1].values()) +
                  sum(v.numel() * 8 for v in host[0][2].values()) for _ in range(1))

        pipe = HostPipeline(torch, R)
        out_hosts = [out_host] + [torch.empty_like(out_host).pin_memory() for _ in range(R - 1)]
        outs = [None] * R

        def e2e_step(i):
            k = i % R
            h, sg = host[k], stage[k]

            def copy_in():
                sg[0].copy_(h[0], non_blocking=True)
                for t in mine:
                    sg[1][t].copy_(h[1][t], non_blocking=True)
                    sg[2][t].copy_(h[2][t], non_blocking=True)

            def run():
                outs[k] = model.forward(sg[0], ebound[k])
                out_hosts[k].copy_(outs[k], non_blocking=True)   # the scores are a few KB: they leave on the same stream

            pipe.step(k, copy_in, run, lambda: None)

        for i in range(2 * R):
            e2e_step(i)
        barrier()
        n_e2e = max(4, min(steps, 10))
        e2e_ms = pipe.timed(e2e_step, n_e2e) / n_e2e
        barrier()
        t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        exchange = form
        results[exchange] = {"samples_per_s": cfg.batch / (float(t[0]) * 1e-3), "ms_per_step": float(t[0]),
                             "e2e_samples_per_s": cfg.batch / (float(t[1]) * 1e-3), "e2e_ms_per_step": float(t[1]),
                             "h2d_bytes_per_step_per_rank": int(h2d), "d2h_bytes_per_step_per_rank": (hi - lo) * 4,
                             "launches_per_step": model.launches_per_step, "cuda_graph": graphed}
        results[exchange].update(checks)
        model.release()
        del model, bound, ebound, devr, stage
        torch.cuda.empty_cache()
    del tables
    torch.cuda.empty_cache()
    return results, {"workload": "DLRM-style: 64 tables x 4,000,000 x 128 uint8 fused rows (table-sharded), batch 4096, "
                                 "bag lengths power-law(1.05) mean 40 max 200, indices power-law(1.05) over rows, "
                                 "int8 rowwise-FC MLPs 256-512-256-128 and 2208-1024-1024-512-1, pairwise-dot "
                                 "interaction; dense layers batch-sharded", "tables": 64, "batch": 4096}


def resnet_measure(torch, dev, steps, cpu_threads=0):
    """ResNet-50 v1.5, fully int8 channelwise-quantized, batch 64 at 224x224x3 (third benchmark
    configuration): images/s with the batch resident in HBM (CUDA-graph replay of the whole
    network) and end to end (fp32 NCHW batch from pinned host memory in, logits out)."""
    from glow_b200 import resnet
    layers = resnet.architecture()
    w = resnet.float_weights(layers)
    g = torch.Generator().manual_seed(7)
    _, ranges = resnet.float_forward(layers, w, torch.randn((16, 3, 224, 224), generator=g), dev)
    q = resnet.quantize_network(layers, w, ranges)
    model = resnet.ResNet50Int8(layers, q, dev)
    host_x = torch.randn((64, 3, 224, 224), generator=g).pin_memory()
    x = host_x.to(dev)
    for _ in range(3):
        out = model.forward(x)
    torch.cuda.synchronize()
    launches = model.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = model.forward(x)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
    torch.cuda.current_stream().wait_stream(side)
    # end to end, two batches in flight: the next batch arrives in a staging buffer while the graph
    # (which reads the fixed buffer x) runs; a device copy moves it into x on the compute stream
    pipe = HostPipeline(torch, 2)
    stages = [torch.empty_like(x) for _ in range(2)]
    outs = [torch.empty_like(out) for _ in range(2)]
    out_hosts = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]

    def e2e(i):
        b = i % 2

        def run():
            x.copy_(stages[b], non_blocking=True)
            graph.replay()
            outs[b].copy_(out, non_blocking=True)

        pipe.step(b, lambda: stages[b].copy_(host_x, non_blocking=True), run,
                  lambda: out_hosts[b].copy_(outs[b], non_blocking=True))

    for i in range(4):
        e2e(i)
    n_e2e = max(4, min(steps, 10))
    e2e_ms = pipe.timed(e2e, n_e2e) / n_e2e
    assert int(model.status.item()) == 0
    ops_per_batch = resnet.conv_ops_per_image(layers) * 64
    cpu = None
    if cpu_threads:
        v, kind, sample = resnet_cpu_rate(layers, q, cpu_threads)
        cpu = {"value": v, "unit": "images/s", "cores": cpu_threads, "kind": kind, "sample": sample}
    return {"metric": "resnet50_int8_images_per_s", "cpu_baseline": cpu, "value": 64 / (ms * 1e-3), "unit": "images/s", "ms_per_batch": ms,
            "e2e_value": 64 / (e2e_ms * 1e-3), "e2e_ms_per_batch": e2e_ms, "h2d_bytes_per_step": host_x.numel() * 4,
            "d2h_bytes_per_step": out.numel() * 4, "launches_per_batch": launches,
            "effective_tops": ops_per_batch / (ms * 1e-3) / 1e12,
            "config": {"workload": "ResNet-50 v1.5 int8: channelwise symmetric filters (He-normal, BN folded), asymmetric "
                                   "int8 activations calibrated on 16 seeded N(0,1) images, int32 bias, batch 64 at "
                                   "224x224x3, every node on the library's kernels", "batch": 64}}


def _cpu_kernels():
    """The reference's libjit compiled here (fast-math build, as Glow ships it) when it was built,
    else the plain-C port: an object with the kernel methods the two model walks below call."""
    from oracle import oracle as orc
    if orc.ref_available("fast"):
        k = orc.LibjitRef("fast")
        return k, "reference", k.channelwise_quantized_conv2d_i8_i32
    orc.lib()
    return orc, "port", orc.conv2d_i8_i32


def resnet_cpu_rate(layers, q, threads, seconds=8.0):
    """ResNet-50 int8 on the host through the reference's own kernels
    (libjit_channelwise_quantized_conv2d_i8_i32, max/avg pool, element add, rowwise FC): one
    224x224 image per host thread, all threads at once -- Glow's CPU backend runs one device per
    core with the batch split (tests/benchmark/Bench.h:54-68).  -> (images/s, kind, sample)."""
    from concurrent.futures import ThreadPoolExecutor
    from glow_b200 import ops
    from oracle import oracle as orc
    k, kind, conv_fn = _cpu_kernels()
    tqp = q["tqp"]
    # libjit's element-wise kernels (add, quantize) are per-element bodies that Glow's JIT wraps in
    # a loop; compiled natively they have no loop of their own, so these two nodes run through the
    # C restatement's loops (the same arithmetic, bit for bit) -- they are a few per cent of the time

    def conv(name, t):
        c = q["conv"][name]
        spec = c["spec"]
        kk, s, p = (spec["k"],) * 2, (spec["stride"],) * 2, (spec["pad"],) * 4
        ohw = ops.conv_out_hw(t.shape[1:3], kk, s, p)
        return conv_fn(t, c["filter"], c["bias"], ohw, kk, s, p, 1, (1, 1), c["out_offset"], c["in_offset"],
                       c["filter_offsets"], c["bias_offsets"], c["params"][:3], c["params"][3:], 1 if spec["relu"] else 0, None)

    def image(seed):
        x = np.random.default_rng(seed).standard_normal((1, 224, 224, 3)).astype(np.float32)
        x = orc.element_quantize_i8(x, *tqp["input"])
        for l in layers:
            if l[0] == "conv":
                x = conv(l[1]["name"], x)
            elif l[0] == "maxpool":
                x = k.max_pool_i8(x, ops.conv_out_hw(x.shape[1:3], (3, 3), (2, 2), (1, 1, 1, 1)), (3, 3), (2, 2), (1, 1, 1, 1),
                                  tqp["conv1"][1])
            elif l[0] == "block":
                y = x
                for c in l[2]:
                    y = conv(c["name"], y)
                sc = conv(l[3]["name"], x) if l[3] else x
                a = q["add"][l[1]]
                out_off = tqp[a["out"]][1]
                x = orc.element_add_i8(y, sc, out_off, tqp[a["lhs"]][1], tqp[a["rhs"]][1], a["lhs_triple"], a["rhs_triple"])
                x = np.maximum(x, np.int8(out_off))  # Relu as max with the offset (CPUMaxSplat)
            elif l[0] == "avgpool":
                src, hw = q["avgpool_in"], x.shape[1]
                tr = ops.quantize_scale_offset_32to8(np.float32(tqp[src][0]) / np.float32(tqp["avgpool"][0]) / np.float32(hw * hw))
                x = k.avg_pool_i8(x, (1, 1), (hw, hw), (1, 1), (0, 0, 0, 0), True, tqp["avgpool"][1], tqp[src][1], tr)
            elif l[0] == "fc":
                f = q["fc"]
                x = k.rowwise_quantized_fc_i8_i32(x.reshape(x.shape[0], -1), f["w"], f["bias"], f["w_offsets"], f["params"][:3],
                                                  f["params"][3:], tqp["fc"][1], tqp[f["in_name"]][1], 0)
        return x

    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(image, range(threads)))  # warm-up pass
        passes, t0 = 0, time.perf_counter()
        while True:
            list(ex.map(image, range(passes * threads, (passes + 1) * threads)))
            passes += 1
            dt = time.perf_counter() - t0
            if dt >= seconds:
                break
    return passes * threads / dt, kind, "%d passes of %d images of 224x224x3 (one per host thread, batch 1 each) in %.1f s" % (
        passes, threads, dt)


def dlrm_cpu_rate(threads, sample=256, tables_timed=4):
    """The recommendation model on the host through the reference's kernels, for a slice of
    `sample` samples: FRWQ-SLS pooling of `tables_timed` of the 64 tables (one libjit call per
    table, tables over the host threads; the cost is linear in the tables, so it is scaled to 64),
    the int8 rowwise-FC MLPs (batch rows over the host threads) and the pairwise-dot interaction.
    -> (samples/s, kind, sample description)."""
    from concurrent.futures import ThreadPoolExecutor
    from glow_b200 import dlrm, ops
    from oracle import oracle as orc
    k, kind, _ = _cpu_kernels()
    cfg = dlrm.DLRMConfig(batch=sample)
    fm = dlrm.float_model(cfg)
    qm = dlrm.quantize_model(cfg, fm, dlrm.fixed_ranges(cfg))
    rng = np.random.default_rng(77)
    tabs = []
    for t in range(tables_timed):
        tab = rng.integers(0, 256, (cfg.rows, cfg.dim + 8), dtype=np.uint8)
        tab[:, cfg.dim:cfg.dim + 4] = rng.uniform(0.001, 0.01, cfg.rows).astype(np.float32).view(np.uint8).reshape(cfg.rows, 4)
        tab[:, cfg.dim + 4:] = rng.uniform(-1, 1, cfg.rows).astype(np.float32).view(np.uint8).reshape(cfg.rows, 4)
        tabs.append(tab)
    dense, lengths, indices = dlrm.make_request(cfg, 31, tables=range(tables_timed))
    dense = dense.numpy()
    pool = k.frwq_slws if kind == "reference" else orc.frwq_slws_u8_f32

    def pool_table(t):
        idx = indices[t].numpy()
        return pool(tabs[t], np.ones(len(idx), np.float32), idx, lengths[t].numpy())

    pool_table(0)  # warm-up
    t0 = time.perf_counter()
    pooled_some = [pool_table(t) for t in range(tables_timed)]
    # one libjit call per table on one thread each; 64 such calls spread over the host threads
    t_pool = (time.perf_counter() - t0) / tables_timed * cfg.tables / min(threads, cfg.tables)
    pooled = np.stack([pooled_some[t % tables_timed] for t in range(cfg.tables)], axis=1)  # [sample, 64, D]
    t0 = time.perf_counter()
    x = orc.element_quantize_i8(dense, *qm["dense_tqp"])
    for fc in qm["bottom"]:
        x = k.rowwise_quantized_fc_i8_i32(x, fc.w, fc.bias, fc.w_offsets, fc.params[:3], fc.params[3:], fc.out_offset,
                                          fc.in_offset, 0, threads=threads)
        if fc.relu:
            x = np.maximum(x, np.int8(fc.out_offset))
    last = qm["bottom"][-1]
    x0 = (x.astype(np.float32) - np.float32(last.out_offset)) * np.float32(last.out_scale)
    z = orc.pairwise_dot_interaction(x0, pooled.reshape(sample, -1).astype(np.float32))
    y = orc.element_quantize_i8(z, *qm["interaction_tqp"])
    for fc in qm["top"]:
        y = k.rowwise_quantized_fc_i8_i32(y, fc.w, fc.bias, fc.w_offsets, fc.params[:3], fc.params[3:], fc.out_offset,
                                          fc.in_offset, 0, threads=threads)
        if fc.relu:
            y = np.maximum(y, np.int8(fc.out_offset))
    t_dense = time.perf_counter() - t0
    return sample / (t_pool + t_dense), kind, (
        "%d of 4096 samples: pooling of %d of the 64 tables timed one thread each and scaled to 64 tables over the host "
        "threads (%.4f s), MLPs and interaction of the slice with the rows over the threads (%.3f s), %d host threads"
        % (sample, tables_timed, t_pool, t_dense, threads))


def run_model_line(args):
    """--workload dlrm | resnet50: the model measurements of the default line's extras, alone."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local)
    sampler.start()
    if args.workload == "dlrm":
        forms = ["local"] if world == 1 else ["fused", "fused_nccl_rendezvous", "nccl"]
        if world == 1 and args.as_rank_of > 1:
            forms = ["emulated"]
        res, cfg = dlrm_measure(torch, dist, dev, rank, world, max(10, args.steps), max(3, args.warmup), forms,
                                as_rank_of=args.as_rank_of)
        best = max(res.values(), key=lambda r: r["samples_per_s"])
        if world == 1 and args.as_rank_of > 1:
            cfg = dict(cfg, as_rank_of=args.as_rank_of,
                       note="one rank's share of a %d-way partition on one GPU: NOT a throughput of the model" % args.as_rank_of)
        line = {"metric": "dlrm_samples_per_s", "value": best["samples_per_s"], "unit": "samples/s", "n_gpus": world,
                "steps": max(10, args.steps), "warmup": max(3, args.warmup), "ms_per_step": best["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8 -> f32 pooling, s8 x s8 -> s32 layers",
                "data": "synthetic", "config": cfg, "by_exchange": res,
                "e2e": {"value": best["e2e_samples_per_s"], "unit": "samples/s",
                        "h2d_bytes_per_step": best["h2d_bytes_per_step_per_rank"] * world,
                        "d2h_bytes_per_step": best["d2h_bytes_per_step_per_rank"] * world},
                "gpu_launches": best["launches_per_step"] * max(10, args.steps)}
        if rank == 0 and not args.no_cpu_baseline:
            v, kind, sample = dlrm_cpu_rate(os.cpu_count() or 1)
            line["cpu_baseline"] = {"value": v, "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": kind, "sample": sample}
    else:
        r = resnet_measure(torch, dev, max(5, args.steps), 0 if args.no_cpu_baseline else (os.cpu_count() or 1))
        line = {"metric": r["metric"], "value": r["value"], "unit": r["unit"], "n_gpus": 1, "steps": max(5, args.steps),
                "warmup": 3, "ms_per_step": r["ms_per_batch"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "s8 x s8 -> s32", "data": "synthetic", "config": r["config"],
                "e2e": {"value": r["e2e_value"], "unit": r["unit"], "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                        "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
                "effective_tops": r["effective_tops"], "gpu_launches": r["launches_per_batch"] * max(5, args.steps)}
        if r.get("cpu_baseline"):
            line["cpu_baseline"] = r["cpu_baseline"]
    line["clocks"] = sampler.stop()
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def slws4_cpu_rate(D, seconds, threads):
    """The fifth configuration's CPU baseline: the reference has no CPU-backend kernel for the
    4-bit kinds, so this times the restatement of its Interpreter kernel (oracle, plain C, one
    call per thread on its own slice of bags) over one 10,000,000-row host table with the
    workload's bag law.  -> (GB/s, passes, seconds)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as orc
    orc.lib()
    rows, line = 10_000_000, D // 2 + 4
    rng = np.random.Generator(np.random.PCG64(0x610B200 + D))
    table = rng.integers(0, 256, (rows, line), dtype=np.uint8)
    so = np.stack([rng.uniform(0.001, 0.01, rows), rng.uniform(-1, 1, rows)], 1).astype(np.float16)
    table[:, D // 2:] = so.view(np.uint8)
    bags = 64          # per thread and pass
    reqs = []
    for r in range(6):
        per = []
        for k in range(threads):
            lengths = rng.poisson(64, bags).astype(np.int32)
            n = int(lengths.sum())
            per.append((lengths, rng.integers(0, rows, n).astype(np.int64), rng.uniform(0, 1, n).astype(np.float16)))
        reqs.append(per)

    def one(job):
        lengths, idx, w = job
        orc.frwq_slws_interp(table, 3, w, idx, lengths, out_fp16=True, fp16_acc=False)
        return int(lengths.sum())

    moved = 0
    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(one, reqs[0]))
        passes, t0 = 0, time.perf_counter()
        while True:
            n = sum(ex.map(one, reqs[(passes + 1) % len(reqs)]))
            moved += n * (line + 8 + 2) + threads * bags * (4 + 2 * D)
            passes += 1
            dt = time.perf_counter() - t0
            if dt >= seconds:
                break
    return moved / dt / 1e9, passes, dt


def slws4_point(torch, ops, dev, D, table_gb, steps):
    """One point of the 4-bit sweep for the default line's extras: the workload of --workload slws4
    (10,000,000-row UInt4FusedFP16QTy tables, 8192 bags per table, Poisson(64) lengths, fp16 weights
    and result) on a smaller set of tables (table_gb, still far larger than L2), device-resident."""
    ROWS4, B = 10_000_000, 8192
    line_bytes = D // 2 + 4
    T = max(1, int(table_gb * 1e9 / (ROWS4 * line_bytes)))
    g = torch.Generator(device=dev).manual_seed(0x610B200 + D)
    tables = []
    for k in range(T):
        t = torch.randint(0, 256, (ROWS4, line_bytes), dtype=torch.uint8, device=dev, generator=g)
        so = torch.stack([torch.empty(ROWS4, device=dev).uniform_(0.001, 0.01, generator=g),
                          torch.empty(ROWS4, device=dev).uniform_(-1, 1, generator=g)], dim=1).to(torch.float16)
        t[:, D // 2:] = so.view(torch.uint8).view(ROWS4, 4)
        tables.append(t)
    del so
    out = torch.empty((T, B, D), dtype=torch.float16, device=dev)
    status = ops.new_status(dev)
    batches, nbytes = [], []
    for r in range(2):
        rng = np.random.Generator(np.random.PCG64(4242 + r))
        lengths = rng.poisson(64, (T, B)).astype(np.int32)
        starts = np.concatenate([[0], np.cumsum(lengths.sum(1))]).astype(np.int64)
        total = int(starts[-1])
        gi = torch.Generator(device=dev).manual_seed(99 + r)
        indices = torch.randint(0, ROWS4, (total,), device=dev, generator=gi)
        weights = torch.rand(total, device=dev, generator=gi).to(torch.float16)
        lengths_d = torch.from_numpy(lengths).to(dev)
        b = ops.SlwsBatch(ops.UINT4_FUSED_FP16, line_bytes, torch.int64, device=dev)
        b.bind(tables, [weights[starts[k]:starts[k + 1]] for k in range(T)],
               [indices[starts[k]:starts[k + 1]] for k in range(T)], [lengths_d[k] for k in range(T)],
               [out[k] for k in range(T)])
        batches.append(b)
        nbytes.append(total * (line_bytes + 8 + 2) + T * B * (4 + 2 * D))
    for i in range(3):
        batches[i % 2].run(status)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        batches[i % 2].run(status)
    e1.record()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ms = e0.elapsed_time(e1)
    gbs = sum(nbytes[i % 2] for i in range(steps)) / (ms * 1e-3) / 1e9
    peak, _ = measured_peak_hbm()
    del tables, batches, out
    torch.cuda.empty_cache()
    return {"dim": D, "value": gbs, "unit": "GB/s", "frac": gbs / peak, "tables": T, "table_gb": T * ROWS4 * line_bytes / 1e9,
            "us_per_launch": ms * 1e3 / steps}


def run_slws4_line(args):
    """--workload slws4: one point of the 4-bit embedding bandwidth sweep (fifth benchmark
    configuration): UInt4FusedFP16QTy tables of 10,000,000 rows x D (D/2 + 4 bytes per row),
    T tables so that they fill --table-gb per GPU, batch 8192 bags per table, lengths
    Poisson(64), uniform int64 indices, fp16 weights U(0,1), fp16 result, fp32 accumulation.
    At N > 1 every rank owns T tables of its own (weak scaling, no collective)."""
    import torch
    import torch.distributed as dist
    from glow_b200 import ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    D, ROWS4, B = args.dim, 10_000_000, 8192
    line_bytes = D // 2 + 4
    T = max(1, int(args.table_gb * 1e9 / (ROWS4 * line_bytes)))
    g = torch.Generator(device=dev).manual_seed(0x610B200 + 77 * rank + D)
    tables = []
    for k in range(T):
        t = torch.randint(0, 256, (ROWS4, line_bytes), dtype=torch.uint8, device=dev, generator=g)
        so = torch.stack([torch.empty(ROWS4, device=dev).uniform_(0.001, 0.01, generator=g),
                          torch.empty(ROWS4, device=dev).uniform_(-1, 1, generator=g)], dim=1).to(torch.float16)
        t[:, D // 2:] = so.view(torch.uint8).view(ROWS4, 4)
        tables.append(t)
    del so
    R = 2
    reqs = []
    for r in range(R):
        rng = np.random.Generator(np.random.PCG64(4242 + 1000 * rank + r))
        lengths = rng.poisson(64, (T, B)).astype(np.int32)
        n = lengths.sum(1)
        starts = np.concatenate([[0], np.cumsum(n)]).astype(np.int64)
        total = int(starts[-1])
        gi = torch.Generator(device=dev).manual_seed(99 + r + 10 * rank)
        indices = torch.randint(0, ROWS4, (total,), device=dev, generator=gi)
        weights = torch.rand(total, device=dev, generator=gi).to(torch.float16)
        reqs.append((torch.from_numpy(lengths).to(dev), indices, weights, starts))
    out = torch.empty((T, B, D), dtype=torch.float16, device=dev)
    status = ops.new_status(dev)
    batches = []
    for lengths_d, indices_d, weights_d, starts in reqs:
        b = ops.SlwsBatch(ops.UINT4_FUSED_FP16, line_bytes, torch.int64, device=dev)
        b.bind(tables, [weights_d[starts[k]:starts[k + 1]] for k in range(T)],
               [indices_d[starts[k]:starts[k + 1]] for k in range(T)], [lengths_d[k] for k in range(T)],
               [out[k] for k in range(T)])
        batches.append(b)
    nbytes = [int(rq[3][-1]) * (line_bytes + 8 + 2) + T * B * (4 + 2 * D) for rq in reqs]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(max(3, args.warmup)):
        batches[i % R].run(status)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        batches[i % R].run(status)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    t_end = time.time() + 1.0
    while len(sampler.lines) < 8 and time.time() < t_end:
        batches[0].run(status)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    assert int(status.item()) == 0
    moved = sum(nbytes[i % R] for i in range(args.steps))
    tm = torch.tensor([ms], dtype=torch.float64, device=dev)
    mv = torch.tensor([moved], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(mv, op=dist.ReduceOp.SUM)
    if rank == 0:
        peak, src = measured_peak_hbm()
        value = float(mv[0]) / (float(tm[0]) * 1e-3) / 1e9
        per_gpu = value / world
        line = {
            "metric": "frwq_slws_4bit_hbm_gbps", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": float(tm[0]) / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u4 -> f32 accumulate -> f16", "data": "synthetic",
            "config": {"workload": "4-bit fused-rowwise SLWS (UInt4FusedFP16QTy): %d tables x 10,000,000 rows x %d cols "
                                   "(%d B rows, %.1f GB per GPU), 8192 bags/table, lengths Poisson(64), uniform int64 "
                                   "indices, fp16 weights and result" % (T, D, line_bytes, T * ROWS4 * line_bytes / 1e9),
                       "dim": D, "tables_per_gpu": T, "l2_policy": "tables far larger than L2, uniform indices"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "peak_source": src,
                         # DRAM bytes per launch: 196 B per row in the ncu capture of a smaller case of D=128
                         # (profiles/), scaled by the rows of a launch; not captured for the other widths
                         "traffic": 196.0 * float(np.mean([int(rq[3][-1]) for rq in reqs])) if D == 128 else None,
                         "kernel": "slws_gather_select_kernel<4,1,1,long,P>",
                         "rows_per_s": sum(int(reqs[i % R][3][-1]) for i in range(args.steps)) / (ms * 1e-3)},
            "gpu_launches": 2 * args.steps, "clocks": clocks}
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, passes, dt = slws4_cpu_rate(D, min(args.cpu_seconds, 10.0), threads)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": "restatement of the reference's Interpreter kernel (the CPU backend has none "
                                              "for 4-bit tables): one 10,000,000-row table, 64 bags per thread per pass, "
                                              "%d passes in %.1f s" % (passes, dt)}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_dyn_fc_line(args):
    """--workload dyn_fc: DynamicRowwiseQuantizedFullyConnected, fp16 [2048, 4096] activations
    N(0,1) x int8 [4096, 4096] weights (held in their [N, K] form), fp16 result.  A step is the row
    quantiser plus the contraction; operations counted are the contraction's 2*M*N*K.  At N > 1
    every rank runs its own batch (replicas)."""
    import torch
    import torch.distributed as dist
    from glow_b200 import ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    M, K, N = 2048, 4096, 4096
    g = torch.Generator(device=dev).manual_seed(0x610B200 + rank)
    R = 8   # rotating inputs and results: 8 x (16 + 16) MB, larger than L2 together with the weights
    xs = [torch.randn((M, K), device=dev, generator=g).to(torch.float16) for _ in range(R)]
    outs = [torch.empty((M, N), dtype=torch.float16, device=dev) for _ in range(R)]
    wt = torch.randint(-127, 128, (N, K), device=dev, generator=g, dtype=torch.int8)
    bias = torch.randn(N, device=dev, generator=g)
    scales = torch.empty(N, device=dev).uniform_(0.001, 0.02, generator=g)
    offsets = torch.zeros(N, dtype=torch.int32, device=dev)
    ws = torch.empty(ops.dynamic_fc_workspace_bytes(M, K, N), dtype=torch.uint8, device=dev)
    status = ops.new_status(dev)

    def step(i):
        ops.dynamic_rowwise_quantized_fc(xs[i % R], None, bias, scales, offsets, weights_transposed=wt,
                                         flags=ops.FC_WEIGHT_OFFSETS_ZERO, out=outs[i % R], workspace=ws, status=status)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    # the K steps as one CUDA graph: two short launches per step would otherwise be paced by the host
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            step(i)
    graph.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    t_end = time.time() + 1.0
    while len(sampler.lines) < 8 and time.time() < t_end:
        step(0)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    assert int(status.item()) == 0
    tm = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    if rank == 0:
        peak, src = measured_peak_int8(ops)
        per_gpu = 2.0 * M * N * K / (float(tm[0]) * 1e-3) / 1e12
        print(json.dumps({
            "metric": "dynamic_quantized_fc_tops", "value": per_gpu * world, "unit": "TOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(tm[0]), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 -> s8 x s8 -> s32 -> f16", "data": "synthetic",
            "config": {"workload": "DynamicRowwiseQuantizedFullyConnected: M=2048 K=4096 N=4096, fp16 activations N(0,1) "
                                   "quantized per row on the device, int8 weights U[-127,127], fp32 bias and column scales",
                       "l2_policy": "8 rotating inputs and results (256 MB) between repeats"},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TOP/s", "frac": per_gpu / peak,
                         "peak_source": src, "traffic": None, "kernel": "dyn_quantize_rows_kernel + i8_gemm_requant_kernel<240,4,2>"},
            "gpu_launches": 2 * args.steps, "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


def run_tbe_line(args):
    """--workload tbe: table-batched embedding bags (IntNBitSplitEmbeddingBags), the shape of the
    reference's tests/benchmark/TBEBench.cpp: T tables of 10,000,000 rows x --dim columns of
    --tbe-type in one byte buffer (rows padded to 16 bytes, scale/offset header first), filling
    --table-gb per GPU; 8192 bags per table, lengths Poisson(64), uniform int64 indices, sum
    pooling, fp16 result.  One launch pools all T * 8192 bags.  At N > 1 every rank owns its own
    tables (weak scaling, no collective)."""
    import torch
    import torch.distributed as dist
    from glow_b200 import ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    D, ROWS, B = args.dim, 10_000_000, 8192
    ty = {"fp16": ops.EST_FLOAT16, "int8": ops.EST_INT8, "int4": ops.EST_INT4}[args.tbe_type]
    row_bytes = ops.split_embedding_row_bytes(D, ty)
    payload = {"fp16": 2 * D, "int8": D + 4, "int4": D // 2 + 4}[args.tbe_type]
    T = max(1, int(args.table_gb * 1e9 / (ROWS * row_bytes)))
    g = torch.Generator(device=dev).manual_seed(0x610B200 + 31 * rank + D)
    weights = torch.empty(T * ROWS * row_bytes, dtype=torch.uint8, device=dev)
    for k in range(T):     # table by table: bounded temporaries
        tab = weights[k * ROWS * row_bytes:(k + 1) * ROWS * row_bytes].view(ROWS, row_bytes)
        if ty == ops.EST_FLOAT16:
            tab.view(torch.float16).normal_(0, 1, generator=g)
        else:
            tab.random_(0, 256, generator=g)
            so = torch.stack([torch.empty(ROWS, device=dev).uniform_(0.001, 0.01, generator=g),
                              torch.empty(ROWS, device=dev).uniform_(-1, 1, generator=g)], dim=1).to(torch.float16)
            tab[:, :4] = so.view(torch.uint8).view(ROWS, 4)
            del so
    placements = torch.full((T,), ops.PLACEMENT_HOST, dtype=torch.int32, device=dev)
    weights_offsets = (torch.arange(T, dtype=torch.int64, device=dev) * (ROWS * row_bytes))
    tys = torch.full((T,), ty, dtype=torch.uint8, device=dev)
    dim_offsets = (torch.arange(T + 1, dtype=torch.int32, device=dev) * D).to(torch.int32)
    R = 2
    reqs = []
    for r in range(R):
        rng = np.random.Generator(np.random.PCG64(777 + 1000 * rank + r))
        lengths = rng.poisson(64, T * B)
        offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
        gi = torch.Generator(device=dev).manual_seed(55 + r + 10 * rank)
        indices = torch.randint(0, ROWS, (int(offsets[-1]),), device=dev, generator=gi)
        reqs.append((indices, torch.from_numpy(offsets).to(dev)))
    out16 = args.tbe_out == "fp16"
    out = torch.empty((B, T * D), dtype=torch.float16 if out16 else torch.float32, device=dev)
    status = ops.new_status(dev)

    def step(i):
        indices, offsets = reqs[i % R]
        ops.int_nbit_split_embedding_bags(weights, weights, placements, weights_offsets, tys, dim_offsets, T * D,
                                          indices, offsets, ops.EP_SUM, out=out, status=status)

    nbytes = [int(rq[0].shape[0]) * (payload + 8) + T * B * (8 + (2 if out16 else 4) * D) for rq in reqs]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    t_end = time.time() + 1.0
    while len(sampler.lines) < 8 and time.time() < t_end:
        step(0)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    assert int(status.item()) == 0
    moved = sum(nbytes[i % R] for i in range(args.steps))
    tm = torch.tensor([ms], dtype=torch.float64, device=dev)
    mv = torch.tensor([moved], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(mv, op=dist.ReduceOp.SUM)
    if rank == 0:
        peak, src = measured_peak_hbm()
        value = float(mv[0]) / (float(tm[0]) * 1e-3) / 1e9
        per_gpu = value / world
        print(json.dumps({
            "metric": "split_embedding_bags_hbm_gbps", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": float(tm[0]) / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "%s -> %s" % (args.tbe_type, "f16 (fp16 running sum, as the reference)" if out16 else "f32"),
            "data": "synthetic",
            "config": {"workload": "IntNBitSplitEmbeddingBags: %d %s tables x 10,000,000 rows x %d cols in one buffer "
                                   "(%d B rows of which %d B are read, %.1f GB per GPU), 8192 bags/table, lengths "
                                   "Poisson(64), uniform int64 indices, sum pooling, %s result"
                                   % (T, args.tbe_type, D, row_bytes, payload, T * ROWS * row_bytes / 1e9, args.tbe_out),
                       "dim": D, "tables_per_gpu": T, "l2_policy": "tables far larger than L2, uniform indices"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "peak_source": src,
                         # DRAM bytes per launch from the ncu captures of smaller cases (profiles/), per row x rows
                         "traffic": ({("int4", 128): 198.0, ("fp16", 128): 264.0}.get((args.tbe_type, D), 0.0) *
                                     float(np.mean([int(rq[0].shape[0]) for rq in reqs]))) or None,
                         "kernel": "split_embedding_bags_kernel<%s,long>" % ("true" if out16 else "false"),
                         "rows_per_s": sum(int(reqs[i % R][0].shape[0]) for i in range(args.steps)) / (ms * 1e-3)},
            "gpu_launches": args.steps, "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


def run_slws4_sharded_line(args):
    """--workload slws4 --shard rows: the 4-bit sweep with every table cut into row ranges over the
    GPUs (rank g holds rows [g*R/G, (g+1)*R/G) of EVERY table).  There are G times as many tables
    as in the unsharded sweep, so each GPU still holds --table-gb of rows; every rank sees the
    whole request, pools its rows into fp32 partial sums that it stores straight into the slab of
    the rank owning the bag, and each rank adds the G slabs and rounds once to fp16.  The value
    is the LOGICAL operator's algorithmic bytes per second (whole tables, whole request)."""
    import torch
    import torch.distributed as dist
    from glow_b200 import ops, sharded
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    D, ROWS4, B = args.dim, 10_000_000, 8192
    line_bytes = D // 2 + 4
    T = max(1, int(args.table_gb * 1e9 / (ROWS4 * line_bytes))) * world      # logical tables
    lo, hi = sharded.row_range(rank, world, ROWS4)
    g = torch.Generator(device=dev).manual_seed(0x610B200 + 77 * rank + D)
    shards = []
    for k in range(T):
        t = torch.randint(0, 256, (hi - lo, line_bytes), dtype=torch.uint8, device=dev, generator=g)
        so = torch.stack([torch.empty(hi - lo, device=dev).uniform_(0.001, 0.01, generator=g),
                          torch.empty(hi - lo, device=dev).uniform_(-1, 1, generator=g)], dim=1).to(torch.float16)
        t[:, D // 2:] = so.view(torch.uint8).view(hi - lo, 4)
        shards.append(t)
    del so
    R = 2
    reqs, logical = [], []
    routed = args.shard == "rows-routed"
    for r in range(R):                                   # the same request on every rank
        rng = np.random.Generator(np.random.PCG64(4242 + r))
        lengths = rng.poisson(64, (T, B)).astype(np.int32)
        starts = np.concatenate([[0], np.cumsum(lengths.sum(1))]).astype(np.int64)
        total = int(starts[-1])
        gi = torch.Generator(device=dev).manual_seed(99 + r)
        indices = torch.randint(0, ROWS4, (total,), device=dev, generator=gi)
        weights = torch.rand(total, device=dev, generator=gi).to(torch.float16).float()   # fp16 values, widened
        logical.append(total)
        if routed:
            # what a front end that routes every index to the GPU owning its row hands this rank:
            # the entries of its rows (local row numbers) and their count per bag
            keep = (indices >= lo) & (indices < hi)
            bag_of = torch.repeat_interleave(torch.arange(T * B, device=dev), torch.from_numpy(lengths.reshape(-1)).to(dev).long())
            sub_len = torch.bincount(bag_of[keep], minlength=T * B).to(torch.int32).view(T, B)
            indices, weights = (indices[keep] - lo).contiguous(), weights[keep].contiguous()
            starts = np.concatenate([[0], np.cumsum(sub_len.sum(1).cpu().numpy())]).astype(np.int64)
            reqs.append((sub_len.contiguous(), indices, weights, starts))
            del keep, bag_of
        else:
            reqs.append((torch.from_numpy(lengths).to(dev), indices, weights, starts))
    nbytes = [n * (line_bytes + 8 + 2) + T * B * (4 + 2 * D) for n in logical]
    results = {}
    checked = {}
    clocks = None
    for form in (["local"] if world == 1 else ["fused", "nccl"]):
        op = sharded.RowShardedSLWS(ops.UINT4_FUSED_FP16, shards, [ROWS4] * T, B, rank, world, exchange=form)
        if form == "fused":
            op.connect_peers()
        pair = []
        for r, (lengths_d, indices_d, weights_d, starts) in enumerate(reqs):
            pair.append(op.prepare([weights_d[starts[k]:starts[k + 1]] for k in range(T)],
                                   [indices_d[starts[k]:starts[k + 1]] for k in range(T)],
                                   [lengths_d[k] for k in range(T)], slab=r if form == "fused" else 0, routed=routed))

        def step(i):
            # request i % 2 is bound to receive slab i % 2, the slab the fused exchange uses at step i
            if form == "fused":
                return op.run(pair)
            return op.run([pair[i % R]])

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        sampler = ClockSampler(local)
        sampler.start()
        op.step = 0
        for i in range(2 * ((max(3, args.warmup) + 1) // 2)):
            step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        t_end = time.time() + 1.0
        while world == 1 and len(sampler.lines) < 8 and time.time() < t_end:
            step(0)
            torch.cuda.synchronize()
        clocks = sampler.stop()
        assert int(op.status.item()) == 0
        tm = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        moved = sum(nbytes[i % R] for i in range(args.steps))
        results[form] = {"gbps": moved / (float(tm[0]) * 1e-3) / 1e9, "ms_per_step": float(tm[0]) / args.steps}
        if world > 1:  # request 0 once more, from step 0 (slab 0), kept for the result checks below
            op.step = 0
            checked[form] = op.run(pair).clone()
            barrier()
        op.release()
        del op, pair
        torch.cuda.empty_cache()
    flags = {}
    if world > 1:
        # Result checks on the real GPUs: the two exchange forms against each other (they add the
        # shards' fp32 partials in different orders, then round once to fp16), and table 0 against
        # the unsharded operator -- its row shards gathered from all ranks, this rank's bags of the
        # logical request pooled by the plain entry point (fp16 result: 2e-3 relative).
        a, b = checked["fused"].float(), checked["nccl"].float()
        forms_ok = bool(torch.allclose(a, b, rtol=4e-3, atol=0.05))
        parts = [torch.empty_like(shards[0]) for _ in range(world)]
        dist.all_gather(parts, shards[0])
        whole = torch.cat(parts, 0)
        rng = np.random.Generator(np.random.PCG64(4242))
        lengths0 = rng.poisson(64, (T, B)).astype(np.int32)
        starts0 = np.concatenate([[0], np.cumsum(lengths0.sum(1))]).astype(np.int64)
        gi = torch.Generator(device=dev).manual_seed(99)
        idx_all = torch.randint(0, ROWS4, (int(starts0[-1]),), device=dev, generator=gi)
        w_all = torch.rand(int(starts0[-1]), device=dev, generator=gi).to(torch.float16)
        per = B // world
        cum = np.concatenate([[0], np.cumsum(lengths0[0])])
        i0, i1 = int(cum[rank * per]), int(cum[(rank + 1) * per])
        want = ops.fused_rowwise_quantized_sparse_lengths_weighted_sum(
            whole, w_all[i0:i1].contiguous(), idx_all[i0:i1].contiguous(),
            torch.from_numpy(lengths0[0, rank * per:(rank + 1) * per].copy()).to(dev), ops.UINT4_FUSED_FP16)
        torch.cuda.synchronize()
        whole_ok = bool(torch.allclose(checked["fused"][0].float(), want.float(), rtol=4e-3, atol=0.05))
        fl = torch.tensor([int(forms_ok), int(whole_ok)], device=dev)
        dist.all_reduce(fl, op=dist.ReduceOp.MIN)
        flags = {"exchange_forms_agree": bool(int(fl[0])), "matches_unsharded": bool(int(fl[1]))}
        del parts, whole, idx_all, w_all
        if not all(flags.values()):
            raise AssertionError("row-sharded results differ: %r" % flags)
    if rank == 0:
        peak, src = measured_peak_hbm()
        best = max(results.values(), key=lambda r: r["gbps"])
        per_gpu = best["gbps"] / world
        print(json.dumps({
            "checks": flags,
            "metric": "frwq_slws_4bit_row_sharded_hbm_gbps", "value": best["gbps"], "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": best["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u4 -> f32 partial sums -> f16", "data": "synthetic",
            "by_exchange": results,
            "config": {"workload": "4-bit fused-rowwise SLWS, tables row-range sharded over the GPUs: %d tables x "
                                   "10,000,000 rows x %d cols (%d B rows, %.1f GB per GPU), 8192 bags/table, lengths "
                                   "Poisson(64), uniform int64 indices, fp16 weights and result; %s"
                                   % (T, D, line_bytes, T * (hi - lo) * line_bytes / 1e9,
                                      "each rank is handed the entries of its own rows" if routed
                                      else "every rank reads the whole request"),
                       "dim": D, "tables": T, "l2_policy": "tables far larger than L2, uniform indices"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "peak_source": src, "traffic": None,
                         "kernel": "slws_gather_select_kernel<4,1,0,long,P,U,sharded> + sum_partials_kernel"},
            "gpu_launches": 3 * args.steps, "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


def workload_config(T):
    return {"workload": "FRWQ-SLWS uint8 fused rows (config 1 law): %d tables x 1,000,000 rows x 64 cols "
                        "(72 B rows), 1024 bags/table, lengths clamp(Poisson(32),1,128), int64 indices, fp32 "
                        "weights, one batched launch per step" % T,
            "tables_per_gpu": T, "rows": ROWS, "dim": DIM, "bags_per_table": BATCH,
            "l2_policy": "inputs larger than L2 (18.4 GB of tables per GPU, indices drawn uniformly)"}


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "int8_fc":
        return run_int8_fc_line(args)
    if args.workload == "slws4":
        return run_slws4_sharded_line(args) if args.shard != "tables" else run_slws4_line(args)
    if args.workload in ("dlrm", "resnet50"):
        return run_model_line(args)
    if args.workload == "tbe":
        return run_tbe_line(args)
    if args.workload == "dyn_fc":
        return run_dyn_fc_line(args)

    import torch
    import torch.distributed as dist
    from glow_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T, R = args.tables, args.requests

    # ---- tables: resident in HBM before anything is timed.  Generated on the device from a
    # seeded torch generator (same value law as workloads.fused_table_u8).
    g = torch.Generator(device=dev).manual_seed(0x610B200 + rank)
    tables = []
    for k in range(T):
        t = torch.randint(0, 256, (ROWS, IN_LINE), dtype=torch.uint8, device=dev, generator=g)
        sc = torch.empty(ROWS, device=dev).uniform_(0.001, 0.01, generator=g)
        of = torch.empty(ROWS, device=dev).uniform_(-1, 1, generator=g)
        t[:, DIM:DIM + 4] = sc.view(torch.uint8).view(ROWS, 4)
        t[:, DIM + 4:] = of.view(torch.uint8).view(ROWS, 4)
        if args.row_bytes:
            t = ops.pad_fused_rows(t, ops.UINT8_FUSED, args.row_bytes)
        tables.append(t)
    del sc, of
    row_line = args.row_bytes or IN_LINE

    # ---- requests: pinned host copies (for the end-to-end leg) and device copies
    host, devr = [], []
    for r in range(R):
        lengths, indices, weights, starts = request_host(T, 99 + 1000 * rank + r)
        hl = torch.from_numpy(lengths).pin_memory()
        hi = torch.from_numpy(indices).pin_memory()
        hw = torch.from_numpy(weights).pin_memory()
        host.append((hl, hi, hw, starts))
        devr.append((hl.to(dev), hi.to(dev), hw.to(dev)))
    max_n = max(int(h[3][T]) for h in host)
    out = torch.empty((T, BATCH, DIM), dtype=torch.float32, device=dev)
    status = ops.new_status(dev)

    def batch_for(lengths_d, indices_d, weights_d, starts):
        b = ops.SlwsBatch(ops.UINT8_FUSED, row_line, torch.int64, device=dev, out_line=DIM)
        b.bind(tables, [weights_d[starts[k]:starts[k + 1]] for k in range(T)],
               [indices_d[starts[k]:starts[k + 1]] for k in range(T)], [lengths_d[k] for k in range(T)],
               [out[k] for k in range(T)])
        return b

    batches = [batch_for(*devr[r], host[r][3]) for r in range(R)]
    bytes_per_step = [algorithmic_bytes(int(host[r][3][T]), T * BATCH) for r in range(R)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    sampler = ClockSampler(local)
    sampler.start()
    for i in range(args.warmup):
        batches[i % R].run(status)
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    ev[0].record()
    for i in range(args.steps):
        batches[i % R].run(status)
        ev[i + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    moved = sum(bytes_per_step[i % R] for i in range(args.steps))
    assert int(status.item()) == 0, "kernel reported invalid input"

    # ---- end to end, through the plug-in's own request call: the tables are static placeholders
    # of a network loaded into the library's device manager, every table's pooling node is an
    # instruction whose indices / weights / lengths are views of three placeholders, and a step is
    # glowb200_device_manager_run_function_async + _wait -- host buffers (pinned, from the device
    # manager) in, pooled result in a host buffer out, copies inside the timed region, two
    # requests in flight over two execution contexts.  Indices cross the host link as int32
    # (tables have fewer than 2^31 rows: Backend::canDoIndexTypeDemotion), and the algorithmic
    # bytes of this leg count them as 4 bytes.
    from glow_b200 import runtime
    max_k = max(int((h[3][1:] - h[3][:-1]).max()) for h in host)
    max_k = (max_k + 63) // 64 * 64          # indices a table's slice has room for
    fn = runtime.Function("frwq_slws_tables")
    tab_ids = [fn.static_placeholder("table%d" % k, ROWS * row_line) for k in range(T)]
    s_idx = fn.placeholder("indices", T * max_k * 4)
    s_w = fn.placeholder("weights", T * max_k * 4)
    s_len = fn.placeholder("lengths", T * BATCH * 4)
    s_out = fn.placeholder("output", T * BATCH * DIM * 4)
    for k in range(T):
        fn.frwq_slws((s_out, k * BATCH * DIM * 4), tab_ids[k], (s_w, k * max_k * 4), (s_idx, k * max_k * 4),
                     (s_len, k * BATCH * 4), kind=ops.UINT8_FUSED, rows=ROWS, in_line=row_line, out_line=DIM,
                     segments=BATCH, num_indices=max_k, idx64=False)
    fn.compile()
    assert fn.batched_pooling_launches == 1
    dm = runtime.DeviceManager(local).init()
    dm.set_context_count(2)
    dm.add_network(fn)
    for k in range(T):  # device-resident hand-over: the tables are already in HBM
        ptr, nb = dm.placeholder_address("frwq_slws_tables", "table%d" % k)
        ops.device_tensor(ptr, (ROWS, row_line), torch.uint8, dev).copy_(tables[k])
    torch.cuda.synchronize()
    e2e_req = []
    for r in range(R):
        hl, hi, hw, starts = host[r]
        bi, bw, bl = dm.io_buffer((T, max_k), np.int32), dm.io_buffer((T, max_k), np.float32), dm.io_buffer((T, BATCH), np.int32)
        bi[:], bw[:] = 0, 0
        bl[:] = hl.numpy()
        hin, hwn = hi.numpy(), hw.numpy()
        for k in range(T):
            n_k = int(starts[k + 1] - starts[k])
            bi[k, :n_k] = hin[starts[k]:starts[k + 1]]
            bw[k, :n_k] = hwn[starts[k]:starts[k + 1]]
        e2e_req.append({"indices": bi, "weights": bw, "lengths": bl})
    NBUF = 2
    out_host = [dm.io_buffer((T, BATCH, DIM), np.float32) for _ in range(NBUF)]
    h2d_step = T * max_k * 8 + T * BATCH * 4
    d2h_step = T * BATCH * DIM * 4

    def e2e_run(n):
        """n requests, two in flight; returns when the last result is in its host buffer."""
        tickets = []
        for i in range(n):
            b = dict(e2e_req[i % R])
            b["output"] = out_host[i % NBUF]
            if i >= NBUF:
                dm.wait(tickets[i - NBUF])   # its output buffer and its context are taken next
            tickets.append(dm.run_function_async("frwq_slws_tables", b, outputs=("output",)))
        for t in tickets[-NBUF:]:
            dm.wait(t)

    e2e_run(2 * NBUF)
    # the plug-in path must give what the kernel ABI gave on the same request
    batches[0].run(status)
    torch.cuda.synchronize()
    dm.wait(dm.run_function_async("frwq_slws_tables", dict(e2e_req[0], output=out_host[0]), outputs=("output",)))
    assert np.array_equal(out_host[0], out.cpu().numpy()), "plug-in request and kernel ABI disagree"
    e2e_steps = max(4, min(args.steps, 20))
    barrier()
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    h2d, d2h = h2d_step * e2e_steps, d2h_step * e2e_steps
    e2e_moved = sum(int(host[i % R][3][T]) * (IN_LINE + 4 + 4) + T * BATCH * (4 + 4 * DIM) for i in range(e2e_steps))
    barrier()
    dm.stop()
    del dm, fn
    # keep the GPU under the same load until the sampler has seen it (a short timed region can
    # fall between two nvidia-smi samples); these extra launches are not timed
    t_end = time.time() + 1.0
    while len(sampler.lines) < 8 and time.time() < t_end:
        for i in range(R):
            batches[i].run(status)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "warm-up, timed steps, end-to-end steps and up to 1 s of the same launches after them"

    # ---- max over ranks
    times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    sums = torch.tensor([moved, e2e_moved], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    total_ms_all, e2e_ms_all = float(times[0]), float(times[1])
    value = float(sums[0]) / (total_ms_all * 1e-3) / 1e9
    e2e_value = float(sums[1]) / (e2e_ms_all * 1e-3) / 1e9

    padded_extra = None
    if world == 1 and not args.no_extras and not args.row_bytes:
        # the same tables stored with rows padded to one 128-byte line each (a loader's choice:
        # costs 78 % more HBM, saves the second line every other 72-byte row straddles); the
        # algorithmic bytes stay those of the 72-byte rows
        wide = [ops.pad_fused_rows(t, ops.UINT8_FUSED, 128) for t in tables]
        pb = []
        for r in range(R):
            lengths_d, indices_d, weights_d = devr[r]
            starts = host[r][3]
            b = ops.SlwsBatch(ops.UINT8_FUSED, 128, torch.int64, device=dev, out_line=DIM)
            b.bind(wide, [weights_d[starts[k]:starts[k + 1]] for k in range(T)],
                   [indices_d[starts[k]:starts[k + 1]] for k in range(T)], [lengths_d[k] for k in range(T)],
                   [out[k] for k in range(T)])
            pb.append(b)
        for i in range(max(3, args.warmup)):
            pb[i % R].run(status)
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for i in range(args.steps):
            pb[i % R].run(status)
        p1.record()
        torch.cuda.synchronize()
        pms = p0.elapsed_time(p1)
        padded_extra = {"metric": METRIC, "value": moved / (pms * 1e-3) / 1e9, "unit": UNIT,
                        "us_per_launch": pms * 1e3 / args.steps, "row_bytes": 128,
                        "note": "same tables, rows padded to 128 B in HBM (32.8 GB instead of 18.4 GB); "
                                "algorithmic bytes counted on the 72-byte rows"}
        del wide, pb
        torch.cuda.empty_cache()

    single_extra = None
    if world == 1 and not args.no_extras:
        # the benchmark definition's own single-node case: ONE table per launch.  The 72 MB table
        # is L2-resident after the first launches, so this is launch latency, not HBM bandwidth.
        lengths_d, indices_d, weights_d = devr[0]
        starts = host[0][3]
        one = ops.SlwsBatch(ops.UINT8_FUSED, row_line, torch.int64, device=dev, out_line=DIM)
        one.bind(tables[:1], [weights_d[:starts[1]]], [indices_d[:starts[1]]], [lengths_d[0]], [out[0]])
        for i in range(10):
            one.run(status)
        torch.cuda.synchronize()
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for i in range(200):
            one.run(status)
        q1.record()
        torch.cuda.synchronize()
        us = q0.elapsed_time(q1) * 1e3 / 200
        # the same 200 launches replayed as one CUDA graph: the device's own latency per launch pair,
        # without the host's call-and-launch pace
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(200):
                one.run(status)
        graph.replay()
        torch.cuda.synchronize()
        q0.record()
        graph.replay()
        q1.record()
        torch.cuda.synchronize()
        us_graph = q0.elapsed_time(q1) * 1e3 / 200
        # the low-latency entry point (a warp per bag) on the same request
        def ll():
            ops.fused_rowwise_quantized_sparse_lengths_weighted_sum(
                tables[0], weights_d[:starts[1]], indices_d[:starts[1]], lengths_d[0], ops.UINT8_FUSED, out=out[0],
                status=status, workspace=one_ws, out_line=DIM, low_latency=True)
        one_ws = torch.empty(ops.slws_workspace_bytes(BATCH, 1), dtype=torch.uint8, device=dev)
        for i in range(10):
            ll()
        graph_ll = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph_ll):
            for i in range(200):
                ll()
        graph_ll.replay()
        torch.cuda.synchronize()
        q0.record()
        graph_ll.replay()
        q1.record()
        torch.cuda.synchronize()
        us_ll_graph = q0.elapsed_time(q1) * 1e3 / 200
        q0.record()
        for i in range(200):
            ll()
        q1.record()
        torch.cuda.synchronize()
        us_ll = q0.elapsed_time(q1) * 1e3 / 200
        single_extra = {"metric": METRIC, "value": algorithmic_bytes(int(starts[1]), BATCH) / (us * 1e-6) / 1e9,
                        "unit": UNIT, "us_per_launch": us, "us_per_launch_in_graph": us_graph,
                        "low_latency_entry_point": {"us_per_launch": us_ll, "us_per_launch_in_graph": us_ll_graph},
                        "note": "one 1,000,000 x 64 table per launch (segments + gather kernels back to back, "
                                "200 launches from the host, then the same 200 as one CUDA graph): the table "
                                "stays in L2, the figure is launch latency"}

    sample_tables = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cpu_threads = os.cpu_count() or 1
        S = min(T, max(cpu_threads, 16))
        sample_tables = [tables[k].cpu().numpy() for k in range(S)]
        if args.row_bytes:  # the CPU reference pools its own layout: dense 72-byte rows
            sample_tables = [np.ascontiguousarray(np.concatenate([t[:, :DIM], t[:, -8:]], axis=1)) for t in sample_tables]
    dlrm_extra = None
    if not args.no_extras:
        # second headline of the same benchmark definition: the recommendation model, all ranks
        del batches, tables, devr, out
        torch.cuda.empty_cache()
        forms = ["local"] if world == 1 else ["fused", "nccl"]
        res, dcfg = dlrm_measure(torch, dist, dev, rank, world, max(10, min(args.steps, 30)), 3, forms)
        best = max(res.values(), key=lambda r: r["samples_per_s"])
        dlrm_extra = {"metric": "dlrm_samples_per_s", "value": best["samples_per_s"], "unit": "samples/s",
                      "n_gpus": world, "scaling": "strong", "e2e_value": best["e2e_samples_per_s"],
                      "by_exchange": res, "config": dcfg}

    if rank == 0:
        peak, peak_src = measured_peak_hbm()
        rows_per_launch = float(np.mean([int(host[r][3][T]) for r in range(R)]))
        launch_us = float(np.mean(step_ms)) * 1e3
        achieved = (moved / args.steps) / (np.mean(step_ms) * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms_all / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(T),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": peak_src,
                         "nominal_peak": 8000.0, "frac_of_nominal": achieved / 8000.0,
                         # DRAM bytes per launch: bytes per gathered row from the ncu capture x the rows
                         "traffic": (None if args.row_bytes else NCU_DRAM_BYTES_PER_ROW * rows_per_launch),
                         "kernel": "slws_gather_select_kernel<8,0,0,long,2,4> (+ slws_segments_from_lengths_kernel, timed together)",
                         "launch_us": launch_us, "algorithmic_bytes_per_launch": moved / args.steps},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d // e2e_steps,
                    "d2h_bytes_per_step": d2h // e2e_steps, "steps": e2e_steps,
                    "ms_per_step": e2e_ms_all / e2e_steps,
                    "call": "glowb200_device_manager_run_function_async + _wait (the request call of the plug-in's "
                            "device manager), two requests in flight over two execution contexts, host wall clock",
                    "host_link": "int32 indices, fp32 weights, int32 lengths in; fp32 pooled rows out; the algorithmic "
                                 "bytes of this leg count 4-byte indices"},
            "gpu_launches": 2 * args.steps,
            "clocks": clocks,
        }
        if dlrm_extra is not None:
            line.setdefault("extras", {})["dlrm"] = dlrm_extra
        if single_extra is not None:
            line.setdefault("extras", {})["slws_single_table"] = single_extra
        if padded_extra is not None:
            line.setdefault("extras", {})["slws_padded_rows"] = padded_extra
        if world == 1 and not args.no_extras:
            # secondary metric of the same benchmark definition: int8 FC throughput
            fc = int8_fc_measure(torch, ops, dev, max(10, min(args.steps, 50)), 3)
            ipeak, isrc = measured_peak_int8(ops)
            line.setdefault("extras", {})["int8_fc"] = {
                "metric": "int8_fc_tops", "value": fc["tops"], "unit": "TOP/s", "us_per_launch": fc["ms"] * 1e3,
                "e2e_value": fc["e2e_tops"], "config": fc_config(),
                "roofline": {"bound": "tensor", "achieved": fc["tops"], "peak": ipeak, "frac": fc["tops"] / ipeak,
                             "peak_source": isrc, "nominal_dense_int8_tops": 4500.0, "frac_of_nominal": fc["tops"] / 4500.0,
                             "library_int8_gemm_tops": fc["library_int8_gemm_tops"]}}
            if not args.no_cpu_baseline:
                tv, tkind, tsample = int8_fc_cpu_rate(4.0, os.cpu_count() or 1)
                line["extras"]["int8_fc"]["cpu_baseline"] = {"value": tv, "unit": "TOP/s", "cores": os.cpu_count() or 1,
                                                             "kind": tkind, "sample": tsample}
        if world == 1 and not args.no_extras:
            line["extras"]["resnet50"] = resnet_measure(torch, dev, max(5, min(args.steps, 20)),
                                                        0 if args.no_cpu_baseline else (os.cpu_count() or 1))
            # the 4-bit sweep, one short point per width (8 GB of tables each; the full-size points
            # are --workload slws4 --dim D)
            line["extras"]["slws_4bit_sweep"] = {
                "metric": "frwq_slws_4bit_hbm_gbps",
                "note": "UInt4FusedFP16QTy, 10,000,000-row tables, 8192 bags of Poisson(64) indices per table, fp16 "
                        "weights and result, fp32 accumulation; 8 GB of tables per point, 10 launches",
                "points": [slws4_point(torch, ops, dev, D, 8.0, 10) for D in (32, 64, 128, 256)]}
        if dlrm_extra is not None and world == 1 and not args.no_cpu_baseline:
            dv, dkind, dsample = dlrm_cpu_rate(os.cpu_count() or 1)
            dlrm_extra["cpu_baseline"] = {"value": dv, "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": dkind,
                                          "sample": dsample}
        if world == 1 and not args.no_cpu_baseline:
            threads, S = cpu_threads, len(sample_tables)
            v, kind, passes, dt = cpu_reference_rate(sample_tables, args.cpu_seconds, threads)
            # Glow's CPU device manager runs one request on one thread and scales by one device per
            # core: the all-thread figure is the baseline, the one-thread figure goes with it
            v1, _, _, _ = cpu_reference_rate(sample_tables[:1], min(3.0, args.cpu_seconds / 4), 1)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": kind, "one_thread_value": v1,
                                    "sample": "first %d of %d tables, %d passes (a different batch each) in %.1f s, one "
                                              "table per libjit call, tables spread over %d host threads"
                                              % (S, T, passes, dt, threads)}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
