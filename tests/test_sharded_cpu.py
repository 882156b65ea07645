"""Host-side logic of row-range sharded embedding tables, on CPU: the row and bag ranges, the
request cut-down, and -- under world_size-2 gloo ranks, with the oracle standing in for the
pooling kernel -- that the shards' partial sums reduce-scattered over the batch give every rank
its slice of the whole table's result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from glow_b200 import sharded, workloads


def test_row_and_bag_ranges_partition():
    for world in (1, 2, 3, 8):
        for rows in (7, 1000, 10_000_019):
            edges = [sharded.row_range(g, world, rows) for g in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == rows
            assert all(edges[g][1] == edges[g + 1][0] for g in range(world - 1))
    assert [sharded.bag_range(g, 4, 64) for g in range(4)] == [(0, 16), (16, 32), (32, 48), (48, 64)]
    with pytest.raises(ValueError):
        sharded.bag_range(0, 3, 64)


def test_bucketize_keeps_order_and_counts():
    lengths = np.array([3, 0, 2, 4], np.int32)
    idx = np.array([5, 50, 7, 60, 1, 99, 8, 55, 2, 1234], np.int64)   # one trailing entry is unused
    w = np.arange(10, dtype=np.float32)
    sub_len, sub_idx, sub_w = sharded.bucketize(lengths, idx, w, 0, 50)
    assert sub_len.tolist() == [2, 0, 1, 2] and sub_idx.tolist() == [5, 7, 1, 8, 2] and sub_w.tolist() == [0, 2, 4, 6, 8]
    sub_len, sub_idx, sub_w = sharded.bucketize(lengths, idx, w, 50, 100)
    assert sub_len.tolist() == [1, 0, 1, 2] and sub_idx.tolist() == [0, 10, 49, 5] and sub_w.tolist() == [1, 3, 5, 7]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
    from oracle import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rows, d, B, kind = 5003, 32, 64, 3
    table = workloads.fused_table_u4(rows, d, seed=77)
    lengths, idx, w = workloads.bags_poisson(B, 20, 0, 60, rows, seed=78, weight_dtype=np.float16)
    lo, hi = sharded.row_range(rank, world, rows)
    sub_len, sub_idx, sub_w = sharded.bucketize(lengths, idx, w, lo, hi)
    # fp32 partial of this shard (the oracle widens the fp16 weights exactly as the kernel's caller does)
    part = oracle.frwq_slws_interp(np.ascontiguousarray(table[lo:hi]), kind, sub_w, sub_idx, sub_len)
    part32 = _partial_fp32(oracle, table[lo:hi], kind, sub_w, sub_idx, sub_len)
    total = torch.from_numpy(part32.copy())
    dist.all_reduce(total)                      # gloo has no reduce-scatter: reduce, then keep my bags
    b0, b1 = sharded.bag_range(rank, world, B)
    mine = total[b0:b1].numpy()
    whole = _partial_fp32(oracle, table, kind, w, idx, lengths)[b0:b1]
    want16 = oracle.frwq_slws_interp(table, kind, w, idx, lengths)[b0:b1].astype(np.float64)
    ok = np.allclose(mine, whole, rtol=1e-5, atol=1e-5) and np.all(
        np.abs(mine.astype(np.float16).astype(np.float64) - want16) <= 2e-3 * np.maximum(np.abs(want16), 1.0))
    ok = ok and part.shape == (B, d)
    open(os.path.join(out_dir, "rank%d" % rank), "w").write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def _partial_fp32(oracle, table, kind, w, idx, lengths):
    """fp32 pooling of an fp16-scale table with fp32 result: dequantised rows from the oracle, summed in fp32."""
    n = int(np.asarray(lengths, np.int64).sum())
    out = np.zeros((len(lengths), (table.shape[1] - 4) * 2), np.float32)
    if n == 0:
        return out
    rows_used = np.ascontiguousarray(table[np.asarray(idx[:n], np.int64)])
    deq = oracle.frwq_slws_interp(rows_used, kind, np.ones(n, np.float16), np.arange(n, dtype=np.int64),
                                  np.ones(n, np.int32)).astype(np.float32)
    terms = deq * np.asarray(w[:n], np.float32)[:, None]
    ends = np.cumsum(np.asarray(lengths, np.int64))
    for i, (s, e) in enumerate(zip(ends - lengths, ends)):
        for j in range(s, e):
            out[i] += terms[j]
    return out


def test_row_range_partials_world2_gloo(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert [open(tmp_path / ("rank%d" % r)).read() for r in range(world)] == ["ok", "ok"]
