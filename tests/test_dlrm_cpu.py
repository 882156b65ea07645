"""Host-side logic of the table-sharded recommendation model, on CPU: the sharding plan and the
all-to-all exchange under world_size-2 gloo ranks must reassemble exactly what an unsharded run
would hand to the dense layers."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from glow_b200 import dlrm


def test_sharding_plan_covers_every_table_once():
    cfg = dlrm.DLRMConfig(tables=13, batch=64)
    for world in (1, 2, 4, 8):
        owned = sorted(t for r in range(world) for t in dlrm.tables_of_rank(cfg, r, world))
        assert owned == list(range(13))
        assert [dlrm.batch_slice(cfg, r, world) for r in range(world)] == [(r * 64 // world, (r + 1) * 64 // world) for r in range(world)]


def test_request_generator_is_seeded_and_in_range():
    cfg = dlrm.DLRMConfig(tables=3, rows=1000, batch=512)
    d1, l1, i1 = dlrm.make_request(cfg, 5)
    d2, l2, i2 = dlrm.make_request(cfg, 5)
    assert torch.equal(d1, d2) and all(torch.equal(l1[t], l2[t]) and torch.equal(i1[t], i2[t]) for t in range(3))
    for t in range(3):
        assert l1[t].dtype == torch.int32 and int(l1[t].max()) <= cfg.max_len and int(l1[t].min()) >= 0
        assert int(l1[t].sum()) == i1[t].shape[0] and int(i1[t].min()) >= 0 and int(i1[t].max()) < cfg.rows
    big = dlrm.DLRMConfig(tables=1, rows=4_000_000, batch=4096)
    _, l, i = dlrm.make_request(big, 1)
    assert 30 < float(l[0].float().mean()) < 50
    # power law over the rows: a small set of hot rows takes a large share of the lookups
    _, counts = torch.unique(i[0], return_counts=True)
    assert counts.max() > 50


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, cfg_kw, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = dlrm.DLRMConfig(**cfg_kw)
    per, D = cfg.batch // world, cfg.dim
    # "pooled" values that encode (bag, table, column) so any misplacement shows
    full = (torch.arange(cfg.batch)[:, None, None] * 10000 + torch.arange(cfg.tables)[None, :, None] * 100 +
            torch.arange(D)[None, None, :]).float()
    mine = dlrm.tables_of_rank(cfg, rank, world)
    send = full[:, mine, :].reshape(world, per, len(mine), D).contiguous()
    got = dlrm.exchange_all_to_all(send, cfg, rank, world)
    lo, hi = dlrm.batch_slice(cfg, rank, world)
    ok = torch.equal(got, full[lo:hi])
    if cfg.tables % world == 0:
        # the pre-allocated form the model's "nccl" exchange takes: equal blocks, one strided copy
        recv = torch.empty(per * cfg.tables * D)
        dist.all_to_all_single(recv, send.view(-1))
        slab = torch.empty((per, cfg.tables, D))
        tl = len(mine)
        slab.view(per, tl, world, D).copy_(recv.view(world, per, tl, D).permute(1, 2, 0, 3))
        ok = ok and torch.equal(slab, full[lo:hi])
    open(os.path.join(out_dir, "rank%d" % rank), "w").write("ok" if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("tables", [4, 5])
def test_all_to_all_exchange_world2_gloo(tmp_path, tables):
    world = 2
    cfg_kw = dict(tables=tables, rows=100, dim=8, batch=12)
    mp.spawn(_worker, args=(world, _free_port(), cfg_kw, str(tmp_path)), nprocs=world, join=True)
    assert [open(tmp_path / ("rank%d" % r)).read() for r in range(world)] == ["ok", "ok"]
