"""Seeded synthetic inputs with the shapes and value laws of the benchmark configurations.

Everything is generated from one master seed with numpy's PCG64; tensor k of a workload uses
stream seed + k.  These stand in for no external dataset: the reference's own benchmarks
(tests/benchmark/SLSBench.cpp, Int8GemmBench.cpp) also run on random data.
"""
import numpy as np

MASTER_SEED = 0x610B200


def _rng(seed, k):
    return np.random.Generator(np.random.PCG64(seed + k))


def fused_table_u8(rows, dim, seed=MASTER_SEED, k=0, fp16_scale_offset=False):
    """uint8 [rows, dim + 8] (or + 4): payload ~U{0..255}, scale ~U(0.001,0.01), offset ~U(-1,1)."""
    r = _rng(seed, k)
    tail = 4 if fp16_scale_offset else 8
    t = np.empty((rows, dim + tail), np.uint8)
    t[:, :dim] = r.integers(0, 256, (rows, dim), dtype=np.uint8)
    sdt = np.float16 if fp16_scale_offset else np.float32
    h = tail // 2
    t[:, dim:dim + h] = r.uniform(0.001, 0.01, rows).astype(sdt).view(np.uint8).reshape(rows, h)
    t[:, dim + h:] = r.uniform(-1, 1, rows).astype(sdt).view(np.uint8).reshape(rows, h)
    return t


def fused_table_u4(rows, dim, seed=MASTER_SEED, k=0, fp16_scale_offset=True):
    """uint8 [rows, dim/2 + 4] (or + 8): packed nibbles ~U{0..255} per byte."""
    r = _rng(seed, k)
    tail = 4 if fp16_scale_offset else 8
    pb = dim // 2
    t = np.empty((rows, pb + tail), np.uint8)
    t[:, :pb] = r.integers(0, 256, (rows, pb), dtype=np.uint8)
    sdt = np.float16 if fp16_scale_offset else np.float32
    h = tail // 2
    t[:, pb:pb + h] = r.uniform(0.001, 0.01, rows).astype(sdt).view(np.uint8).reshape(rows, h)
    t[:, pb + h:] = r.uniform(-1, 1, rows).astype(sdt).view(np.uint8).reshape(rows, h)
    return t


def bags_poisson(batch, mean, lo, hi, rows, seed=MASTER_SEED, k=1, index_dtype=np.int64, weight_dtype=np.float32):
    """lengths = clamp(Poisson(mean), lo, hi) int32; indices uniform over rows; weights ~U(0,1)."""
    r = _rng(seed, k)
    lengths = np.clip(r.poisson(mean, batch), lo, hi).astype(np.int32)
    n = int(lengths.sum())
    indices = r.integers(0, rows, n).astype(index_dtype)
    weights = r.uniform(0, 1, n).astype(weight_dtype)
    return lengths, indices, weights


def config1(seed=MASTER_SEED, rows=1_000_000, dim=64, batch=1024, k=0):
    """Single FRWQ-SLWS node: 1M x 64 uint8 table (72 B rows), 1024 bags of Poisson(32) in [1,128]."""
    table = fused_table_u8(rows, dim, seed, 10 * k)
    lengths, indices, weights = bags_poisson(batch, 32, 1, 128, rows, seed, 10 * k + 1)
    return table, weights, indices, lengths


def slws_algorithmic_bytes(num_indices, segments, in_line, out_line, index_bytes=8, weight_bytes=4, out_elem_bytes=4):
    """Bytes one launch must move: rows + indices + weights, plus lengths and the result
    (the accounting of tests/benchmark/CommonSLSEB.h:120-176, with the real index width)."""
    return num_indices * (in_line + index_bytes + weight_bytes) + segments * (4 + out_line * out_elem_bytes)


def config2(seed=MASTER_SEED, M=2048, K=4096, N=4096):
    """Int8 rowwise-quantized FullyConnected.  Returns a dict of numpy arrays and scalars."""
    r = _rng(seed, 100)
    return dict(
        inp=r.integers(-128, 128, (M, K), dtype=np.int8),
        w=r.integers(-127, 128, (N, K), dtype=np.int8),
        w_scales=r.uniform(0.001, 0.02, N).astype(np.float32),
        w_offsets=np.zeros(N, np.int32),
        bias=r.integers(-2 ** 16, 2 ** 16 + 1, N).astype(np.int32),
        in_scale=np.float32(0.05), in_offset=3, out_scale=np.float32(0.5), out_offset=0,
        # the benchmark definition leaves the bias type open; fixed here: scale = in_scale * mean weight scale, offset 0
        bias_scale=np.float32(5e-4), bias_offset=0)
