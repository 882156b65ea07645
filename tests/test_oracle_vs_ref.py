"""Our C restatement against pytorch/glow's own libjit sources compiled unmodified
(oracle/_ref/libjit_strict.so): bit for bit on seeded inputs."""
import numpy as np
import pytest


def _table_u8(rng, rows, d):
    t = np.empty((rows, d + 8), np.uint8)
    t[:, :d] = rng.integers(0, 256, (rows, d), dtype=np.uint8)
    t[:, d:d + 4] = rng.uniform(0.001, 0.01, rows).astype(np.float32).view(np.uint8).reshape(rows, 4)
    t[:, d + 4:] = rng.uniform(-1, 1, rows).astype(np.float32).view(np.uint8).reshape(rows, 4)
    return t


@pytest.mark.parametrize("d", [1, 3, 64, 128, 200])
@pytest.mark.parametrize("idt", [np.int64, np.int32])
def test_frwq_slws_u8(oracle, libjit_ref, d, idt):
    rng = np.random.default_rng(100 + d)
    rows, B = 5000, 96
    t = _table_u8(rng, rows, d)
    lengths = np.clip(rng.poisson(12, B), 0, 50).astype(np.int32)
    lengths[3] = 0
    n = int(lengths.sum())
    idx = rng.integers(0, rows, n + 7).astype(idt)  # trailing indices are ignored
    w = rng.uniform(0, 1, n + 7).astype(np.float32)
    want = libjit_ref.frwq_slws(t, w, idx, lengths)
    np.testing.assert_array_equal(oracle.frwq_slws_u8_f32(t, w, idx, lengths).view(np.uint32), want.view(np.uint32))
    # the Interpreter form of the same kind performs the same float operations
    np.testing.assert_array_equal(oracle.frwq_slws_interp(t, 0, w, idx, lengths).view(np.uint32), want.view(np.uint32))


def test_fast_math_build_is_within_tolerance(oracle, libjit_ref):
    if not oracle.ref_available("fast"):
        pytest.skip("fast flavour not built")
    fast = oracle.LibjitRef("fast")
    rng = np.random.default_rng(7)
    t = _table_u8(rng, 20000, 64)
    lengths = np.clip(rng.poisson(32, 256), 1, 128).astype(np.int32)
    n = int(lengths.sum())
    idx = rng.integers(0, 20000, n).astype(np.int64)
    w = rng.uniform(0, 1, n).astype(np.float32)
    a, b = libjit_ref.frwq_slws(t, w, idx, lengths), fast.frwq_slws(t, w, idx, lengths)
    assert np.max(np.abs(a - b) / np.maximum(np.abs(a), 1.0)) < 1e-5


@pytest.mark.parametrize("has_end", [False, True])
def test_embedding_bag(oracle, libjit_ref, has_end):
    rng = np.random.default_rng(21)
    rows, B, d = 3000, 40, 64
    t = _table_u8(rng, rows, d)
    lengths = rng.integers(0, 20, B)
    offs = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    n = int(offs[-1])
    idx = rng.integers(0, rows, n).astype(np.int32)
    w = rng.uniform(-1, 1, n).astype(np.float32)
    o = offs if has_end else offs[:-1]
    want = libjit_ref.embedding_bag_byte_rowwise_offsets(t, w, idx, o, has_end)
    got = oracle.embedding_bag_byte_rowwise_offsets(t, 0, w, idx, o, has_end)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def _triples(oracle, rng, n):
    pre, post, sc = [], [], []
    for s in np.exp(rng.uniform(np.log(1e-5), np.log(3.0), n)).astype(np.float32):
        a, b, c = oracle.quantize_scale_offset_32to8(s)
        pre.append(a); post.append(b); sc.append(c)
    return [np.array(x, np.int32) for x in (pre, post, sc)]


def test_scale32_matches_libjit_rescale(oracle, libjit_ref):
    """libjit_scale is not exported; libjit_element_rescale_kernel_i8 wraps it."""
    rng = np.random.default_rng(3)
    src = rng.integers(-128, 128, 400).astype(np.int8)
    for _ in range(25):
        pre, post, sc = (int(x[0]) for x in _triples(oracle, rng, 1))
        io, oo = int(rng.integers(-20, 20)), int(rng.integers(-20, 20))
        np.testing.assert_array_equal(oracle.element_rescale_i8(src, oo, io, (pre, post, sc)),
                                      libjit_ref.element_rescale_i8(src, oo, io, (pre, post, sc)))


@pytest.mark.parametrize("M,K,N", [(7, 33, 5), (32, 256, 48), (3, 1000, 130)])
@pytest.mark.parametrize("w_off_zero", [True, False])
def test_rowwise_quantized_fc(oracle, libjit_ref, M, K, N, w_off_zero):
    rng = np.random.default_rng(M * 1000 + N)
    inp = rng.integers(-128, 128, (M, K)).astype(np.int8)
    w = rng.integers(-127, 128, (N, K)).astype(np.int8)
    bias = rng.integers(-2 ** 16, 2 ** 16, N).astype(np.int32)
    w_off = np.zeros(N, np.int32) if w_off_zero else rng.integers(-30, 30, N).astype(np.int32)
    ws = rng.uniform(0.001, 0.02, N).astype(np.float32)
    p = oracle.rowwise_requant_params(ws, 0.05, 5e-4, 0.5)
    args = (inp, w, bias, w_off, p[:3], p[3:], 0, 3, 0)
    want = libjit_ref.rowwise_quantized_fc_i8_i32(*args)
    np.testing.assert_array_equal(oracle.rowwise_quantized_fc_i8_i32(*args), want)
    np.testing.assert_array_equal(oracle.rowwise_quantized_fc_i8_i32(*args, threads=3), want)
    assert len(np.unique(want)) > 20  # not saturated: the comparison means something


def test_fc_and_matmul(oracle, libjit_ref):
    rng = np.random.default_rng(8)
    M, K, N = 9, 77, 21
    inp = rng.integers(-128, 128, (M, K)).astype(np.int8)
    w = rng.integers(-128, 128, (K, N)).astype(np.int8)
    bias = rng.integers(-5000, 5000, N).astype(np.int32)
    bt = oracle.quantize_scale_offset_32to8(np.float32(0.002) / (np.float32(0.05) * np.float32(0.01)))
    ot = oracle.quantize_scale_offset_32to8(np.float32(0.05) * np.float32(0.01) / np.float32(0.3))
    want = libjit_ref.fc_i8_i32(inp, w, bias, -4, 3, 2, 1, bt, ot)
    np.testing.assert_array_equal(oracle.fc_i8_i32(inp, w, bias, -4, 3, 2, 1, bt, ot), want)
    want = libjit_ref.matmul_i8(inp, w, 5, -3, 7, ot)
    np.testing.assert_array_equal(oracle.matmul_i8(inp, w, 5, -3, 7, ot), want)


CONV_CASES = [
    # n, ih, iw, ic, oc, k, stride, pad, group, dil, act
    (2, 9, 9, 8, 16, (3, 3), (1, 1), (1, 1, 1, 1), 1, (1, 1), 0),
    (1, 12, 10, 6, 8, (3, 3), (2, 2), (1, 1, 1, 1), 2, (1, 1), 1),
    (2, 8, 8, 16, 32, (1, 1), (1, 1), (0, 0, 0, 0), 1, (1, 1), 1),
    (1, 15, 15, 3, 8, (7, 7), (2, 2), (3, 3, 3, 3), 1, (1, 1), 0),
    (1, 5, 5, 8, 8, (3, 3), (1, 1), (1, 1, 1, 1), 8, (1, 1), 2),
    (1, 11, 11, 4, 4, (3, 3), (1, 1), (2, 2, 2, 2), 1, (2, 2), 5),
]


def _out_hw(ih, iw, k, s, p, d):
    oh = (ih + p[0] + p[2] - ((k[0] - 1) * d[0] + 1)) // s[0] + 1
    ow = (iw + p[1] + p[3] - ((k[1] - 1) * d[1] + 1)) // s[1] + 1
    return oh, ow


@pytest.mark.parametrize("case", CONV_CASES)
def test_channelwise_conv(oracle, libjit_ref, case):
    n, ih, iw, ic, oc, k, s, p, g, d, act = case
    rng = np.random.default_rng(ic * 100 + oc)
    inp = rng.integers(-128, 128, (n, ih, iw, ic)).astype(np.int8)
    filt = rng.integers(-127, 128, (oc, k[0], k[1], ic // g)).astype(np.int8)
    bias = rng.integers(-3000, 3000, oc).astype(np.int32)
    fo = rng.integers(-3, 4, oc).astype(np.int32)
    bo = rng.integers(-5, 5, oc).astype(np.int32)
    fs = rng.uniform(0.002, 0.02, oc).astype(np.float32)
    in_scale, out_scale = np.float32(0.04), np.float32(0.9)
    pp = oracle.rowwise_requant_params(fs, in_scale, in_scale * fs, out_scale)
    act_args = {2: [-20, 60], 5: list(oracle.quantize_scale_offset_32to8(0.1))}.get(act)
    ohw = _out_hw(ih, iw, k, s, p, d)
    args = (inp, filt, bias, ohw, k, s, p, g, d, 4, -2, fo, bo, pp[:3], pp[3:], act, act_args)
    want = libjit_ref.channelwise_quantized_conv2d_i8_i32(*args)
    np.testing.assert_array_equal(oracle.conv2d_i8_i32(*args), want)
    assert len(np.unique(want)) > 10
    # per-tensor form
    t1 = [int(x[0]) for x in pp[:3]]
    t2 = [int(x[0]) for x in pp[3:]]
    unroll = 8 if (oc // g) % 8 == 0 else 1
    want = libjit_ref.conv2d_i8_i32(inp, filt, bias, ohw, k, s, p, g, d, 4, -2, int(fo[0]), int(bo[0]), t1, t2, act,
                                    act_args, depth_unroll=unroll)
    got = oracle.conv2d_i8_i32(inp, filt, bias, ohw, k, s, p, g, d, 4, -2, fo[:1], bo[:1], t1, t2, act, act_args,
                               per_channel=False)
    np.testing.assert_array_equal(got, want)


def test_pools_and_elementwise(oracle, libjit_ref):
    rng = np.random.default_rng(13)
    x = rng.integers(-128, 128, (2, 11, 9, 5)).astype(np.int8)
    for k, s, p in [((3, 3), (2, 2), (1, 1, 1, 1)), ((2, 2), (2, 2), (0, 0, 0, 0)), ((7, 7), (1, 1), (3, 3, 3, 3))]:
        ohw = _out_hw(11, 9, k, s, p, (1, 1))
        np.testing.assert_array_equal(oracle.max_pool_i8(x, ohw, k, s, p, -7), libjit_ref.max_pool_i8(x, ohw, k, s, p, -7))
        for cip in (True, False):
            area = k[0] * k[1]
            tr = oracle.quantize_scale_offset_32to8(np.float32(0.03) / np.float32(0.05) / (np.float32(area) if cip else np.float32(1)))
            np.testing.assert_array_equal(oracle.avg_pool_i8(x, ohw, k, s, p, cip, 3, -4, tr),
                                          libjit_ref.avg_pool_i8(x, ohw, k, s, p, cip, 3, -4, tr))
    a = rng.integers(-128, 128, 500).astype(np.int8)
    b = rng.integers(-128, 128, 500).astype(np.int8)
    lt = oracle.quantize_scale_offset_32to8(0.7)
    rt = oracle.quantize_scale_offset_32to8(1.9)
    np.testing.assert_array_equal(oracle.element_add_i8(a, b, 5, -3, 9, lt, rt),
                                  libjit_ref.element_add_i8(a, b, 5, -3, 9, lt, rt))
    np.testing.assert_array_equal(oracle.element_relu_i8(a, -10, 4, lt), libjit_ref.element_relu_i8(a, -10, 4, lt))
    f = (rng.standard_normal(600) * 3).astype(np.float32)
    f[:8] = [0.5 * 0.05, 1.5 * 0.05, 2.5 * 0.05, -0.5 * 0.05, -1.5 * 0.05, 1000.0, -1000.0, 0.0]
    np.testing.assert_array_equal(oracle.element_quantize_i8(f, 0.05, 3), libjit_ref.element_quantize_i8(f, 0.05, 3))


@pytest.mark.parametrize("d", [1, 5, 64, 130])
@pytest.mark.parametrize("idt", [np.int64, np.int32])
def test_plain_and_rowwise_quantized_slws(oracle, libjit_ref, d, idt):
    rng = np.random.default_rng(300 + d)
    rows, B = 4000, 80
    lengths = np.clip(rng.poisson(10, B), 0, 40).astype(np.int32)
    lengths[5] = 0
    n = int(lengths.sum())
    idx = rng.integers(0, rows, n).astype(idt)
    w = rng.uniform(-1, 1, n).astype(np.float32)
    table = rng.normal(0, 1, (rows, d)).astype(np.float32)
    for weights in (w, None):
        want = libjit_ref.sparse_lengths_weighted_sum(table, weights, idx, lengths)
        got = (oracle.sparse_lengths_weighted_sum_f32(table, w, idx, lengths) if weights is not None
               else oracle.sparse_lengths_sum_f32(table, idx, lengths))
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    q = rng.integers(0, 256, (rows, d), dtype=np.uint8)
    sc, off = rng.uniform(0.001, 0.01, rows).astype(np.float32), rng.uniform(-1, 1, rows).astype(np.float32)
    want = libjit_ref.rowwise_quantized_slws(q, sc, off, w, idx, lengths)
    got = oracle.rowwise_quantized_slws_f32(q, sc, off, w, idx, lengths)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("bins", [0, 1, 10, 2000])
def test_quantization_profile_vs_libjit(oracle, libjit_ref, bins):
    """Running min / max and histogram over several tensors with growing, shrinking and constant
    ranges: the restatement against libjit_quantization_profile, bit for bit."""
    rng = np.random.default_rng(12 + bins)
    ci_o = np.array([np.finfo(np.float32).max, np.finfo(np.float32).min], np.float32)
    ci_r, h_o, h_r = ci_o.copy(), np.zeros(bins, np.float32), np.zeros(bins, np.float32)
    for step, (scale, shift, n) in enumerate([(1.0, 0.0, 5000), (0.3, 0.1, 777), (4.0, -2.0, 9000), (4.0, 5.0, 3000),
                                              (0.0, 1.5, 100), (20.0, 0.0, 1)]):
        x = (rng.normal(0, 1, n) * scale + shift).astype(np.float32)
        ci_o, h_o = oracle.quantization_profile(x, ci_o, h_o)
        ci_r, h_r = libjit_ref.quantization_profile(x, ci_r, h_r)
        np.testing.assert_array_equal(ci_o.view(np.uint32), ci_r.view(np.uint32))
        np.testing.assert_array_equal(h_o.view(np.uint32), h_r.view(np.uint32))
    if bins:
        assert h_o.sum() == 5000 + 777 + 9000 + 3000 + 100 + 1


def test_binary_muldiv_batched_add_vs_libjit(oracle, libjit_ref):
    """The remaining arithmetic mini-kernels (sub / max / min, mul / div) and BatchedAdd (int8 and
    int32 slice): the restatement against libjit, bit for bit."""
    rng = np.random.default_rng(31)
    a = rng.integers(-128, 128, 700).astype(np.int8)
    b = rng.integers(-128, 128, 700).astype(np.int8)
    lt, rt = oracle.quantize_scale_offset_32to8(0.7), oracle.quantize_scale_offset_32to8(1.9)
    for op in range(4):
        np.testing.assert_array_equal(oracle.element_binary_i8(op, a, b, 5, -3, 9, lt, rt),
                                      libjit_ref.element_binary_i8(op, a, b, 5, -3, 9, lt, rt))
    np.testing.assert_array_equal(oracle.element_binary_i8(0, a, b, 5, -3, 9, lt, rt), oracle.element_add_i8(a, b, 5, -3, 9, lt, rt))
    tm = oracle.quantize_scale_offset_32to8(0.011)
    np.testing.assert_array_equal(oracle.element_muldiv_i8(False, a, b, 2, -3, 9, tm), libjit_ref.element_muldiv_i8(False, a, b, 2, -3, 9, tm))
    td = oracle.quantize_scale_offset_32to8(3.3)
    b_nz = np.where(b == 9, np.int8(10), b)            # the reference divides by (rhs - rhsOffset)
    np.testing.assert_array_equal(oracle.element_muldiv_i8(True, a, b_nz, 2, -3, 9, td), libjit_ref.element_muldiv_i8(True, a, b_nz, 2, -3, 9, td))
    batch = rng.integers(-128, 128, (13, 40)).astype(np.int8)
    for sl in (rng.integers(-128, 128, 40).astype(np.int8), rng.integers(-100000, 100000, 40).astype(np.int32)):
        st = oracle.quantize_scale_offset_32to8(0.004 if sl.dtype == np.int32 else 1.3)
        np.testing.assert_array_equal(oracle.batched_add_i8(batch, sl, -6, 4, 1, lt, st), libjit_ref.batched_add_i8(batch, sl, -6, 4, 1, lt, st))
