"""Parity of the table-batched embedding bags (IntNBitSplitEmbeddingBags and its weighted form)
through the C ABI: the sixteen cases of the reference's own operator tests, and seeded random
requests over tables of mixed element type, bit for bit against the oracle (the kernel keeps the
Interpreter's accumulation order and rounds an fp16 result after every row as it does)."""
import numpy as np
import pytest
import torch

from glow_b200 import ops
from split_embedding_cases import CASES, case_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def run_gpu(a, so_fp32=False, row_alignment=16, status=None):
    iw = a.get("indice_weights")
    out = ops.int_nbit_split_embedding_bags(
        t(a["dev_weights"]), t(a["uvm_weights"]), t(a["placements"]), t(a["weights_offsets"]), t(a["weights_tys"]),
        t(a["dim_offsets"]), a["total_dims"], t(a["indices"]), t(a["offsets"]), a["pooling_mode"],
        indice_weights=None if iw is None else t(iw),
        out_dtype=torch.float16 if a["out_fp16"] else torch.float32, scale_offset_is_fp32=so_fp32,
        row_alignment=row_alignment, status=status)
    return out.cpu().numpy()


def bits(x):
    return x.view(np.uint16 if x.dtype == np.float16 else np.uint32)


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("idt", [np.int32, np.int64])
def test_reference_unit_cases(oracle, name, idt):
    a, expected, tol = case_inputs(name, idt)
    st = ops.new_status(DEV)
    got = run_gpu(a, status=st)
    np.testing.assert_allclose(got.astype(np.float32), expected, atol=tol, rtol=0)
    np.testing.assert_array_equal(bits(got), bits(oracle.int_nbit_split_embedding_bags(**a)))
    assert int(st.item()) == 0


def random_tables(rng, specs, so_fp32, align, first_at=0):
    """specs: (weights_ty, num_dims, rows, placement).  Returns the two byte buffers (tables are
    written to the one their placement selects; the other holds noise there), and the arrays
    describing them."""
    so = 4 if so_fp32 else 2
    at, offs, chunks = first_at, [], []
    for ty, d, rows, _ in specs:
        rb = ops.split_embedding_row_bytes(d, ty, scale_offset_is_fp32=so_fp32, row_alignment=align)
        tab = rng.integers(0, 256, (rows, rb), dtype=np.uint8)
        if ty == ops.EST_FLOAT:
            tab[:, :4 * d] = rng.normal(0, 1, (rows, d)).astype(np.float32).view(np.uint8)
        elif ty == ops.EST_FLOAT16:
            tab[:, :2 * d] = rng.normal(0, 1, (rows, d)).astype(np.float16).view(np.uint8)
        else:
            sdt = np.float32 if so_fp32 else np.float16
            hdr = np.stack([rng.uniform(0.001, 0.02, rows), rng.uniform(-1, 1, rows)], 1).astype(sdt)
            tab[:, :2 * so] = hdr.view(np.uint8)
        offs.append(at)
        chunks.append(tab.reshape(-1))
        at += tab.size
    total = at + 16   # slack: the last column of an odd-width int4 row sits one byte past its payload
    dev = rng.integers(0, 256, total, dtype=np.uint8)
    uvm = rng.integers(0, 256, total, dtype=np.uint8)
    for (ty, d, rows, placement), o, c in zip(specs, offs, chunks):
        (dev if placement == ops.PLACEMENT_HOST else uvm)[o:o + c.size] = c
    return dev, uvm, np.array(offs, np.int64)


def random_request(rng, specs, B, mean_len, idt):
    lens = rng.poisson(mean_len, (len(specs), B))
    lens[:, B // 3] = 0
    offsets = np.concatenate([[0], np.cumsum(lens.reshape(-1))]).astype(idt)
    idx = np.concatenate([rng.integers(0, rows, int(lens[i].sum())) for i, (_, _, rows, _) in enumerate(specs)])
    return idx.astype(idt), offsets


MIXED = [(ops.EST_INT8, 64, 3000, 3), (ops.EST_INT4, 128, 2000, 1), (ops.EST_FLOAT, 20, 500, 1),
         (ops.EST_FLOAT16, 36, 800, 3), (ops.EST_INT4, 30, 900, 2), (ops.EST_INT8, 1, 100, 3),
         (ops.EST_INT8, 300, 400, 1), (ops.EST_FLOAT, 130, 300, 3), (ops.EST_FLOAT16, 513, 200, 1),
         (ops.EST_INT4, 1100, 150, 3), (ops.EST_INT4, 7, 50, 1), (ops.EST_INT8, 252, 600, 3)]


@pytest.mark.parametrize("out16", [False, True])
@pytest.mark.parametrize("weighted", [None, np.float32, np.float16])
@pytest.mark.parametrize("pooling", [ops.EP_SUM, ops.EP_MEAN])
@pytest.mark.parametrize("idt,wo_dt", [(np.int32, np.int32), (np.int64, np.int64)])
def test_mixed_tables_bit_exact(oracle, out16, weighted, pooling, idt, wo_dt):
    rng = np.random.default_rng(1000 + 2 * int(out16) + pooling)
    dev, uvm, offs = random_tables(rng, MIXED, False, 16)
    B = 97
    idx, offsets = random_request(rng, MIXED, B, 9, idt)
    dims = np.array([0] + [d for _, d, _, _ in MIXED], np.int64).cumsum().astype(np.int32)
    a = dict(dev_weights=dev, uvm_weights=uvm, placements=np.array([p for *_, p in MIXED], np.int32),
             weights_offsets=offs.astype(wo_dt), weights_tys=np.array([s[0] for s in MIXED], np.uint8),
             dim_offsets=dims, total_dims=int(dims[-1]), indices=idx, offsets=offsets, pooling_mode=pooling,
             out_fp16=out16, indice_weights=None)
    if weighted is not None:
        a["indice_weights"] = rng.uniform(-1, 1, idx.size).astype(weighted)
    st = ops.new_status(DEV)
    got = run_gpu(a, status=st)
    want = oracle.int_nbit_split_embedding_bags(**a)
    np.testing.assert_array_equal(bits(got), bits(want))
    assert int(st.item()) == 0


@pytest.mark.parametrize("so_fp32", [False, True])
@pytest.mark.parametrize("align,first_at", [(16, 0), (4, 4), (1, 3), (64, 64), (8, 24)])
def test_row_alignments_and_fp32_headers(oracle, so_fp32, align, first_at):
    """Rows padded to other alignments, tables at odd byte offsets (the byte-wise load path), and
    fp32 scale/offset headers; columns no table covers stay zero."""
    rng = np.random.default_rng(77 + align)
    specs = [(ops.EST_INT8, 40, 500, 3), (ops.EST_INT4, 66, 400, 3), (ops.EST_FLOAT16, 9, 300, 1),
             (ops.EST_FLOAT, 5, 200, 1), (ops.EST_INT4, 15, 100, 3)]
    dev, uvm, offs = random_tables(rng, specs, so_fp32, align, first_at)
    idx, offsets = random_request(rng, specs, 50, 6, np.int32)
    dims = np.array([0] + [d for _, d, _, _ in specs], np.int64).cumsum().astype(np.int32)
    a = dict(dev_weights=dev, uvm_weights=uvm, placements=np.array([p for *_, p in specs], np.int32),
             weights_offsets=offs.astype(np.int32), weights_tys=np.array([s[0] for s in specs], np.uint8),
             dim_offsets=dims, total_dims=int(dims[-1]) + 3, indices=idx, offsets=offsets, pooling_mode=ops.EP_SUM,
             out_fp16=False, indice_weights=rng.uniform(0, 1, idx.size).astype(np.float32))
    st = ops.new_status(DEV)
    got = run_gpu(a, so_fp32=so_fp32, row_alignment=align, status=st)
    want = oracle.int_nbit_split_embedding_bags(so_fp32=so_fp32, row_alignment=align, **a)
    np.testing.assert_array_equal(bits(got), bits(want))
    assert not got[:, -3:].any()
    assert int(st.item()) == 0


def test_bad_rows_and_tables_are_reported():
    rng = np.random.default_rng(5)
    specs = [(ops.EST_INT8, 32, 100, 3), (ops.EST_INT8, 32, 100, 3), (ops.EST_INT8, 32, 100, 0)]
    dev, uvm, offs = random_tables(rng, specs, False, 16)
    B = 4
    idx = np.zeros(3 * B * 2, np.int32)
    idx[1] = 10 ** 6      # far outside the buffer
    idx[2] = -1
    offsets = np.arange(0, 3 * B * 2 + 1, 2, dtype=np.int32)
    tys = np.array([ops.EST_INT8, 4, ops.EST_INT8], np.uint8)   # table 1: int2, table 2: device placement
    a = dict(dev_weights=dev, uvm_weights=uvm, placements=np.array([3, 3, 0], np.int32),
             weights_offsets=offs.astype(np.int32), weights_tys=tys,
             dim_offsets=np.array([0, 32, 64, 96], np.int32), total_dims=96, indices=idx, offsets=offsets,
             pooling_mode=ops.EP_SUM, out_fp16=False, indice_weights=None)
    st = ops.new_status(DEV)
    got = run_gpu(a, status=st)
    assert int(st.item()) == (ops.STATUS_INDEX_OUT_OF_RANGE | ops.STATUS_UNSUPPORTED_TABLE)
    assert not got[:, 32:].any()
    # bag 0 lost its second row, bag 1 its first; the rest are two copies of row 0
    so = dev[:4].view(np.float16).astype(np.float32)
    row0 = dev[4:36].astype(np.float32) * so[0] + so[1]
    np.testing.assert_array_equal(got[0, :32], row0)
    np.testing.assert_array_equal(got[2, :32], row0 + row0)


def test_empty_request():
    z32 = torch.zeros(0, dtype=torch.int32, device=DEV)
    out = ops.int_nbit_split_embedding_bags(
        torch.zeros(16, dtype=torch.uint8, device=DEV), torch.zeros(16, dtype=torch.uint8, device=DEV),
        t(np.array([3], np.int32)), t(np.array([0], np.int32)), t(np.array([2], np.uint8)),
        t(np.array([0, 4], np.int32)), 4, z32, t(np.zeros(4, np.int32)))
    assert out.shape == (3, 4) and not out.any()


def test_properties_on_large_tables():
    """Sizes the oracle does not reach in seconds (three tables, 8.5 M rows, 0.9 GB; 12,288 bags of
    about 50 rows): properties that hold bit for bit whatever the size -- weights of 1 equal the
    unweighted operator, a power-of-two weight scales an fp32 result exactly, mean pooling is the
    sum divided by the bag length, and the batched launch equals one launch per table."""
    g = torch.Generator(device=DEV).manual_seed(11)
    specs = [(ops.EST_INT4, 128, 4_000_000), (ops.EST_INT8, 64, 3_000_000), (ops.EST_FLOAT16, 96, 1_500_000)]
    B = 4096
    parts, offs, at = [], [], 0
    for ty, d, rows in specs:
        rb = ops.split_embedding_row_bytes(d, ty)
        tab = torch.randint(0, 256, (rows, rb), dtype=torch.uint8, device=DEV, generator=g)
        if ty == ops.EST_FLOAT16:
            tab.view(torch.float16).normal_(0, 1, generator=g)
        else:
            so = torch.stack([torch.empty(rows, device=DEV).uniform_(0.001, 0.01, generator=g),
                              torch.empty(rows, device=DEV).uniform_(-1, 1, generator=g)], 1).to(torch.float16)
            tab[:, :4] = so.view(torch.uint8).view(rows, 4)
        offs.append(at)
        parts.append(tab.reshape(-1))
        at += tab.numel()
    weights = torch.cat(parts)
    T = len(specs)
    tys = t(np.array([s[0] for s in specs], np.uint8))
    place = t(np.full(T, ops.PLACEMENT_HOST, np.int32))
    wo = t(np.array(offs, np.int64))
    dims = np.array([0] + [d for _, d, _ in specs]).cumsum().astype(np.int32)
    D = int(dims[-1])
    rng = np.random.default_rng(2)
    lens = rng.poisson(50, (T, B))
    offsets_h = np.concatenate([[0], np.cumsum(lens.reshape(-1))]).astype(np.int64)
    idx = torch.cat([torch.randint(0, rows, (int(lens[i].sum()),), device=DEV, generator=g)
                     for i, (_, _, rows) in enumerate(specs)])
    offsets = t(offsets_h)
    st = ops.new_status(DEV)

    def run(pool=ops.EP_SUM, iw=None, dt=torch.float32):
        return ops.int_nbit_split_embedding_bags(weights, weights, place, wo, tys, t(dims), D, idx, offsets, pool,
                                                 indice_weights=iw, out_dtype=dt, status=st)

    base = run()
    assert torch.isfinite(base).all() and base.abs().max() > 1
    ones = torch.ones(idx.numel(), device=DEV)
    assert torch.equal(run(iw=ones), base)
    assert torch.equal(run(iw=ones * 0.25), base * 0.25)
    n = torch.from_numpy(lens.T.astype(np.float32)).to(DEV)                      # [B, T]
    per_col = torch.repeat_interleave(n, torch.tensor([d for _, d, _ in specs], device=DEV), dim=1)
    want_mean = torch.where(per_col > 0, base / per_col.clamp(min=1), base)
    assert torch.equal(run(pool=ops.EP_MEAN), want_mean)
    base16 = run(dt=torch.float16)
    assert torch.equal(run(iw=ones.to(torch.float16), dt=torch.float16), base16)
    # one launch per table
    for i, (ty, d, rows) in enumerate(specs):
        lo, hi = int(offsets_h[i * B]), int(offsets_h[(i + 1) * B])
        single = ops.int_nbit_split_embedding_bags(
            weights, weights, place[i:i + 1], wo[i:i + 1], tys[i:i + 1], t(np.array([0, d], np.int32)), d,
            idx[lo:hi], t(offsets_h[i * B:(i + 1) * B + 1] - lo), ops.EP_SUM, status=st)
        assert torch.equal(single, base[:, int(dims[i]):int(dims[i + 1])])
    assert int(st.item()) == 0
