"""Parity of the embedding operators beside the fused gather-pool: plain and rowwise-quantized
SparseLengths(Weighted)Sum (bit for bit with the oracle: same accumulation order, no FMA), the
fused-rowwise quantiser on the device (same bytes as the oracle), and row-range sharded pooling
(partials of the shards against the oracle on each shard's rows; their sum against the whole
table within the fp32 / fp16 tolerances of the operator)."""
import numpy as np
import pytest
import torch

from glow_b200 import ops, sharded, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def make_table(seed, rows, d, kind):
    make = workloads.fused_table_u8 if kind < 2 else workloads.fused_table_u4
    return make(rows, d, seed=seed, fp16_scale_offset=bool(kind & 1))


def _request(rng, rows, B, mean, idt, extra=0):
    lengths = np.clip(rng.poisson(mean, B), 0, 4 * mean).astype(np.int32)
    lengths[B // 3] = 0
    n = int(lengths.sum())
    idx = rng.integers(0, rows, n + extra).astype(idt)
    w = rng.uniform(-1, 1, n + extra).astype(np.float32)
    return lengths, idx, w


@pytest.mark.parametrize("d", [1, 3, 16, 64, 128, 132, 520, 1030])
@pytest.mark.parametrize("idt", [np.int64, np.int32])
def test_sparse_lengths_sums_fp32_table(oracle, d, idt):
    rng = np.random.default_rng(40 + d)
    rows, B = 6000, 300
    lengths, idx, w = _request(rng, rows, B, 14, idt, extra=5)
    table = rng.normal(0, 1, (rows, d)).astype(np.float32)
    st = ops.new_status(DEV)
    got = ops.sparse_lengths_weighted_sum(t(table), t(w), t(idx), t(lengths), status=st).cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32),
                                  oracle.sparse_lengths_weighted_sum_f32(table, w, idx, lengths).view(np.uint32))
    got = ops.sparse_lengths_sum(t(table), t(idx), t(lengths), status=st).cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), oracle.sparse_lengths_sum_f32(table, idx, lengths).view(np.uint32))
    assert int(st.item()) == 0


@pytest.mark.parametrize("d", [2, 7, 64, 128, 260])
@pytest.mark.parametrize("idt", [np.int64, np.int32])
def test_rowwise_quantized_slws(oracle, d, idt):
    rng = np.random.default_rng(80 + d)
    rows, B = 5000, 257
    lengths, idx, w = _request(rng, rows, B, 20, idt)
    q = rng.integers(0, 256, (rows, d), dtype=np.uint8)
    sc, off = rng.uniform(0.001, 0.01, rows).astype(np.float32), rng.uniform(-1, 1, rows).astype(np.float32)
    st = ops.new_status(DEV)
    got = ops.rowwise_quantized_sparse_lengths_weighted_sum(t(q), t(sc), t(off), t(w), t(idx), t(lengths),
                                                            status=st).cpu().numpy()
    want = oracle.rowwise_quantized_slws_f32(q, sc, off, w, idx, lengths)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    assert int(st.item()) == 0


def test_unfused_sums_report_bad_indices_and_lengths():
    rng = np.random.default_rng(3)
    table = rng.normal(0, 1, (100, 8)).astype(np.float32)
    lengths = np.array([2, 3], np.int32)
    idx = np.array([1, 100, 5, -1, 7], np.int64)
    st = ops.new_status(DEV)
    got = ops.sparse_lengths_sum(t(table), t(idx), t(lengths), status=st).cpu().numpy()
    assert int(st.item()) & ops.STATUS_INDEX_OUT_OF_RANGE
    np.testing.assert_array_equal(got[0], table[1])          # the bad rows are skipped
    np.testing.assert_array_equal(got[1], table[5] + table[7])
    st = ops.new_status(DEV)
    ops.sparse_lengths_sum(t(table), t(idx[:3]), t(lengths), status=st)
    assert int(st.item()) & ops.STATUS_LENGTHS_OVERRUN


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("cols", [2, 8, 64, 130])
def test_fused_rowwise_quantize_on_device(oracle, kind, cols):
    rng = np.random.default_rng(11 * kind + cols)
    table = rng.normal(0, 1, (700, cols)).astype(np.float32)
    table[5] = 0.25          # constant row: scale 1
    table[6, 0] = 1e4        # wide range
    got = ops.fused_rowwise_quantize(t(table), kind).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.fused_rowwise_quantize(table, kind))


def test_quantize_then_pool_round_trip(oracle):
    """Float table -> device quantiser -> fused gather-pool, against the float table's own pooling."""
    rng = np.random.default_rng(17)
    rows, B, d = 20000, 512, 64
    table = rng.normal(0, 1, (rows, d)).astype(np.float32)
    lengths, idx, w = _request(rng, rows, B, 24, np.int64)
    w = np.abs(w)
    fused = ops.fused_rowwise_quantize(t(table), 0)
    got = ops.fused_rowwise_quantized_sparse_lengths_weighted_sum(fused, t(w), t(idx), t(lengths), 0).cpu().numpy()
    want = oracle.sparse_lengths_weighted_sum_f32(table, w, idx, lengths)
    # every value moves by at most half a quantisation step of its row: (max-min)/255/2
    step = (table.max(1) - table.min(1)) / 255.0
    bound = np.zeros((B, 1))
    ends = np.cumsum(lengths)
    for i, (s, e) in enumerate(zip(ends - lengths, ends)):
        bound[i] = (w[s:e] * step[idx[s:e]] * 0.5).sum()
    assert np.all(np.abs(got - want) <= bound * 1.001 + 1e-4)


def test_sum_partials():
    rng = np.random.default_rng(2)
    parts = rng.normal(0, 1, (5, 333, 7)).astype(np.float32)
    want = parts[0].copy()
    for g in range(1, 5):
        want += parts[g]
    got = ops.sum_partials(t(parts)).cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    got16 = ops.sum_partials(t(parts), torch.float16).cpu().numpy()
    np.testing.assert_array_equal(got16.view(np.uint16), want.astype(np.float16).view(np.uint16))


def unpack(table, kind):
    """(q [rows, D], scale [rows, 1], offset [rows, 1]) of a fused table, as float64."""
    tail = 4 if kind & 1 else 8
    pay = table[:, :-tail]
    if kind >= 2:
        q = np.empty((table.shape[0], pay.shape[1] * 2), np.float64)
        q[:, 0::2], q[:, 1::2] = pay & 0xF, pay >> 4
    else:
        q = pay.astype(np.float64)
    so = table[:, -tail:].copy().view(np.float16 if kind & 1 else np.float32).astype(np.float64)
    return q, so[:, :1], so[:, 1:]


def pooled_f64(table, kind, w, idx, lengths, full_scale=False):
    """The operator in float64 straight from the table's bytes.  full_scale=True gives what the
    fp32 comparisons scale with instead: sum_j |w_j| * (|scale_j| * qmax + |offset_j|), the size of
    a row's terms before anything cancels.  (A shard's bag is often one or two rows; if their
    value happens to cancel to ~0 it has no meaningful relative error of its own.)"""
    n = int(np.asarray(lengths, np.int64).sum())
    rows = np.asarray(idx[:n], np.int64)
    q, sc, off = unpack(table[rows], kind)
    wv = np.asarray(w[:n], np.float64)[:, None]
    terms = np.abs(wv) * (np.abs(sc) * (15.0 if kind >= 2 else 255.0) + np.abs(off)) * np.ones_like(q) if full_scale \
        else wv * (q * sc + off)
    out = np.zeros((len(lengths), q.shape[1]))
    ends = np.cumsum(np.asarray(lengths, np.int64))
    for i, (s, e) in enumerate(zip(ends - lengths, ends)):
        out[i] = terms[s:e].sum(0)
    return out


def oracle_result(oracle, table, kind, w32, idx, lengths):
    """The oracle's operator on the request: fp32 for the fp32-scale kinds, fp16 (fp32 accumulation,
    fp16 weights and result, as the reference types the node) for the fp16-scale kinds."""
    w = w32.astype(np.float16) if kind & 1 else w32
    return oracle.frwq_slws_interp(np.ascontiguousarray(table), kind, w, idx, np.asarray(lengths, np.int32)).astype(np.float64)


def close(got, want, scale, rel):
    return np.all(np.abs(got - want) <= rel * np.maximum(scale, np.abs(want)) + 1e-30)


@pytest.mark.parametrize("kind,d", [(0, 64), (3, 128), (3, 32), (1, 64), (2, 256)])
@pytest.mark.parametrize("shards", [2, 3, 8])
def test_row_range_shards(oracle, kind, d, shards):
    """Every shard pools only its own rows of the table; the partials sum to the whole."""
    rng = np.random.default_rng(1000 * kind + d + shards)
    rows, B = 30011, 384
    table = make_table(1000 * kind + d + shards, rows, d, kind)
    lengths = np.clip(rng.poisson(30, B), 0, 100).astype(np.int32)
    lengths[::7] *= 4                                     # some long bags
    n = int(lengths.sum())
    idx = rng.integers(0, rows, n).astype(np.int64)
    w32 = rng.uniform(0, 1, n).astype(np.float16).astype(np.float32)   # fp16-representable weights
    dev_idx, dev_len, dev_w = t(idx), t(lengths), t(w32)
    partials = torch.empty((shards, B, d), dtype=torch.float32, device=DEV)
    st = ops.new_status(DEV)
    rel = 2e-3 if kind & 1 else 1e-5                      # the oracle's result is fp16 for the fp16 kinds
    for g in range(shards):
        lo, hi = sharded.row_range(g, shards, rows)
        batch = ops.SlwsBatch(kind, table.shape[1])
        batch.bind([t(table[lo:hi])], [dev_w], [dev_idx], [dev_len], [partials[g]], row_ranges=[(lo, rows)])
        batch.run(status=st)
        torch.cuda.synchronize()
        got = partials[g].cpu().numpy().astype(np.float64)
        # this shard against the oracle on the request cut down to the shard's rows ...
        sub_len, sub_idx, sub_w = sharded.bucketize(lengths, idx, w32, lo, hi)
        scale = pooled_f64(table[lo:hi], kind, sub_w, sub_idx, sub_len, full_scale=True)
        assert close(got, oracle_result(oracle, table[lo:hi], kind, sub_w, sub_idx, sub_len), scale, rel)
        # ... and, at fp32 accuracy for every kind, against the same sum in float64
        assert close(got, pooled_f64(table[lo:hi], kind, sub_w, sub_idx, sub_len), scale, 1e-5)
    assert int(st.item()) == 0
    scale = pooled_f64(table, kind, w32, idx, lengths, full_scale=True)
    total = ops.sum_partials(partials).cpu().numpy().astype(np.float64)
    assert close(total, pooled_f64(table, kind, w32, idx, lengths), scale, 1e-5)
    want = oracle_result(oracle, table, kind, w32, idx, lengths)
    out = ops.sum_partials(partials, torch.float16 if kind & 1 else torch.float32).cpu().numpy().astype(np.float64)
    assert close(out, want, scale, rel)


def test_row_range_reports_indices_outside_the_whole_table():
    rng = np.random.default_rng(5)
    table = make_table(5, 1000, 64, 0)
    lengths = np.array([3, 2], np.int32)
    idx = np.array([10, 900, 1000, 20, -1], np.int64)      # 1000 and -1 are outside the whole table
    w = np.ones(5, np.float32)
    out = torch.zeros((2, 64), dtype=torch.float32, device=DEV)
    st = ops.new_status(DEV)
    ops.SlwsBatch(0, 72).bind([t(table[:500])], [t(w)], [t(idx)], [t(lengths)], [out], row_ranges=[(0, 1000)]).run(status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == ops.STATUS_INDEX_OUT_OF_RANGE
    st = ops.new_status(DEV)
    ops.SlwsBatch(0, 72).bind([t(table[:500])], [t(w[:2])], [t(idx[:2])], [t(np.array([2], np.int32))], [out[:1]],
                              row_ranges=[(0, 1000)]).run(status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0                              # row 900 is another shard's: no report


@pytest.mark.parametrize("kind,d", [(3, 64), (0, 64), (3, 256)])
@pytest.mark.parametrize("world", [1, 2, 4])
def test_row_sharded_operator(oracle, kind, d, world):
    """RowShardedSLWS end to end (ranks emulated in one process): every rank's [T, B/G, D] slice
    against the oracle's result on the whole tables."""
    T, rows, B = 3, [20011, 9973, 15000], 256
    tables = [make_table(900 + 10 * kind + i, rows[i], d, kind) for i in range(T)]
    reqs = [workloads.bags_poisson(B, 24, 0, 80, rows[i], seed=950 + i, weight_dtype=np.float16) for i in range(T)]
    dev_w = [t(w.astype(np.float32)) for _, _, w in reqs]
    dev_idx = [t(idx) for _, idx, _ in reqs]
    dev_len = [t(ln) for ln, _, _ in reqs]
    ranks = []
    for g in range(world):
        shards = [t(tables[i][slice(*sharded.row_range(g, world, rows[i]))]) for i in range(T)]
        ranks.append(sharded.RowShardedSLWS(kind, shards, rows, B, g, world, exchange="emulated" if world > 1 else "local"))
    if world == 1:
        outs = [ranks[0].run_request(dev_w, dev_idx, dev_len)]
    else:
        for r in ranks:
            r.set_peers(ranks)
        for r in ranks:
            r.pool(r.prepare(dev_w, dev_idx, dev_len))
        outs = [r.reduce() for r in ranks]
    torch.cuda.synchronize()
    assert all(int(r.status.item()) == 0 for r in ranks)
    got = torch.cat(outs, dim=1).cpu().numpy().astype(np.float64)          # [T, B, D]
    assert outs[0].dtype == (torch.float16 if kind & 1 else torch.float32)
    for i in range(T):
        ln, idx, w = reqs[i]
        w32 = w.astype(np.float32)
        scale = pooled_f64(tables[i], kind, w32, idx, ln, full_scale=True)
        assert close(got[i], oracle_result(oracle, tables[i], kind, w32, idx, ln), scale, 2e-3 if kind & 1 else 1e-5)
        if not kind & 1:
            continue
        # fp16 result = one rounding of the fp32-accurate sum
        exact = pooled_f64(tables[i], kind, w32, idx, ln)
        assert np.all(np.abs(got[i] - exact) <= 1e-5 * scale + np.abs(exact) * 2.0 ** -11 + 1e-30)


@pytest.mark.parametrize("kind,d,row_bytes", [(0, 64, 128), (0, 64, 80), (0, 128, 256), (3, 128, 128), (2, 64, 64),
                                              (1, 64, 96), (0, 20, 32)])
def test_padded_rows_pool_identically(oracle, kind, d, row_bytes):
    """A table re-laid with padded rows (payload, zeros, scale/offset last) gives the bits the dense
    table gives, and what the oracle gives when it is told the padded line size."""
    rng = np.random.default_rng(70 + d + kind)
    rows, B = 9000, 300
    table = make_table(31 + kind, rows, d, kind)
    lengths, idx, w = _request(rng, rows, B, 20, np.int64)
    wd = np.float16 if kind & 1 else np.float32
    dt, dw, di, dl = t(table), t(np.abs(w).astype(wd)), t(idx), t(lengths)
    padded = ops.pad_fused_rows(dt, kind, row_bytes)
    assert padded.shape == (rows, row_bytes)
    host = padded.cpu().numpy()
    tail = 4 if kind & 1 else 8
    np.testing.assert_array_equal(host[:, :table.shape[1] - tail], table[:, :-tail])
    np.testing.assert_array_equal(host[:, -tail:], table[:, -tail:])
    assert not host[:, table.shape[1] - tail:-tail].any()
    st = ops.new_status(DEV)
    dense = ops.fused_rowwise_quantized_sparse_lengths_weighted_sum(dt, dw, di, dl, kind, status=st)
    wide = ops.fused_rowwise_quantized_sparse_lengths_weighted_sum(padded, dw, di, dl, kind, status=st, out_line=d)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and torch.equal(dense, wide)
    if kind == 0:   # the CPU kernel's own addressing of a wide row: columns first, scale/offset last
        want = oracle.frwq_slws_u8_f32(host, np.abs(w), idx, lengths, out_line=d)
        scale = pooled_f64(table, kind, np.abs(w), idx, lengths, full_scale=True)
        assert close(wide.cpu().numpy().astype(np.float64), want.astype(np.float64), scale, 1e-5)
