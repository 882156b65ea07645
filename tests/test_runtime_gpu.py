"""The host runtime on a GPU: the reference's DeviceManager conformance cases
(tests/unittests/DeviceManagerTest.cpp:132-973: Basic, MultiRun, MultiFunction, AvailableMemory,
eviction and lookup errors, partial tensors) transposed to quantized functions, with every
result checked against the CPU oracle."""
import numpy as np
import pytest

from glow_b200 import ops, runtime, workloads
from glow_b200._lib import GlowB200Error

pytestmark = pytest.mark.gpu


@pytest.fixture()
def dm():
    d = runtime.DeviceManager(0).init()
    yield d
    d.stop()


def slws_function(name, table, segments, max_indices):
    rows, in_line = table.shape
    f = runtime.Function(name)
    data = f.constant(name + "_data", table)
    w = f.placeholder(name + "_weights", max_indices * 4)
    idx = f.placeholder(name + "_indices", max_indices * 8)
    ln = f.placeholder(name + "_lengths", segments * 4)
    out = f.placeholder(name + "_output", segments * (in_line - 8) * 4)
    f.frwq_slws(out, data, w, idx, ln, kind=ops.UINT8_FUSED, rows=rows, in_line=in_line, out_line=in_line - 8,
                segments=segments, num_indices=max_indices)
    return f.compile()


def run_slws(dm, name, w, idx, lengths, segments, dim, max_indices):
    out = np.zeros((segments, dim), np.float32)
    wp = np.zeros(max_indices, np.float32); wp[:w.size] = w
    ip = np.zeros(max_indices, np.int64); ip[:idx.size] = idx
    dm.run_function(name, {name + "_weights": wp, name + "_indices": ip, name + "_lengths": lengths.copy(),
                           name + "_output": out})
    return out


def test_basic_and_multi_run(oracle, dm):
    table = workloads.fused_table_u8(5000, 64, 1, 0)
    f = slws_function("main", table, 128, 128 * 40)
    dm.add_network(f)
    for seed in (1, 2, 3):  # MultiRun: the same function, different requests
        lengths, idx, w = workloads.bags_poisson(128, 20, 0, 40, 5000, seed, 1)
        got = run_slws(dm, "main", w, idx, lengths, 128, 64, 128 * 40)
        want = oracle.frwq_slws_u8_f32(table, w, idx, lengths)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


def test_multi_function_memory_accounting_and_errors(oracle, dm):
    t1, t2 = workloads.fused_table_u8(3000, 64, 5, 0), workloads.fused_table_u8(2000, 64, 6, 0)
    f1, f2 = slws_function("func1", t1, 32, 640), slws_function("func2", t2, 32, 640)
    total = dm.available_memory
    assert total == dm.maximum_memory
    dm.add_network(f1)
    after1 = dm.available_memory
    assert total - after1 >= t1.nbytes
    dm.add_network(f2)
    assert dm.available_memory < after1
    with pytest.raises(GlowB200Error, match="already have a function called func1") as e:
        dm.add_network(f1)
    assert e.value.code == runtime.RUNTIME_ERROR
    for name, t in (("func1", t1), ("func2", t2)):
        lengths, idx, w = workloads.bags_poisson(32, 10, 0, 20, t.shape[0], 9, 1)
        np.testing.assert_allclose(run_slws(dm, name, w, idx, lengths, 32, 64, 640), oracle.frwq_slws_u8_f32(t, w, idx, lengths),
                                   rtol=1e-5, atol=1e-5)
    with pytest.raises(GlowB200Error) as e:
        dm.run_function("nope", {})
    assert e.value.code == runtime.NET_NOT_FOUND
    dm.evict_network("func1")
    dm.evict_network("func2")
    assert dm.available_memory == total
    with pytest.raises(GlowB200Error) as e:
        dm.evict_network("func1")
    assert e.value.code == runtime.NET_NOT_FOUND
    dm.add_network(f1)  # a function can come back after eviction (ReuseModule)
    assert dm.available_memory == after1


def test_out_of_device_memory_is_an_error_not_a_crash():
    small = runtime.DeviceManager(0, 1 << 20).init()
    f = slws_function("big", workloads.fused_table_u8(50000, 64, 2, 0), 16, 160)
    with pytest.raises(GlowB200Error) as e:
        small.add_network(f)
    assert e.value.code == runtime.OUT_OF_DEVICE_MEMORY
    assert small.available_memory == 1 << 20
    small.stop()


def test_invalid_sparse_input_becomes_a_runtime_error(dm):
    table = workloads.fused_table_u8(100, 64, 3, 0)
    dm.add_network(slws_function("chk", table, 4, 16))
    lengths = np.array([2, 2, 0, 0], np.int32)
    with pytest.raises(GlowB200Error, match="invalid sparse input") as e:
        run_slws(dm, "chk", np.ones(4, np.float32), np.array([1, 2, 100, 3], np.int64), lengths, 4, 64, 16)
    assert e.value.code == runtime.RUNTIME_ERROR
    # the device manager stays usable and the status word was cleared
    got = run_slws(dm, "chk", np.ones(4, np.float32), np.array([1, 2, 4, 3], np.int64), lengths, 4, 64, 16)
    assert np.isfinite(got).all() and got[:2].any()


def test_partial_tensor_binding(oracle, dm):
    """A binding shorter than its placeholder is a partial tensor: the rest reads as zero."""
    table = workloads.fused_table_u8(1000, 64, 4, 0)
    dm.add_network(slws_function("part", table, 8, 64))
    lengths = np.array([3, 2, 0, 0, 0, 0, 0, 0], np.int32)
    idx = np.array([5, 6, 7, 8, 9], np.int64)
    w = np.ones(5, np.float32)
    out = np.zeros((8, 64), np.float32)
    dm.run_function("part", {"part_weights": w, "part_indices": idx, "part_lengths": lengths[:2].copy(), "part_output": out})
    np.testing.assert_allclose(out, oracle.frwq_slws_u8_f32(table, w, idx, lengths), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("quantize_first", [False, True])
def test_quantized_network_bit_exact(oracle, dm, quantize_first):
    """NCHW fp32 -> Transpose -> Quantize (or Quantize -> Transpose, the order Glow's optimizer leaves:
    the runtime then makes one kernel of the pair) -> conv3x3+Relu -> MaxPool -> [conv1x1, shortcut] -> Add -> Relu
    -> AvgPool -> rowwise FC -> Dequantize, every integer parameter derived by the runtime's compile()."""
    rng = np.random.default_rng(12)
    n, cin, hw, c1, c2, classes = 3, 16, 12, 32, 32, 10
    f = runtime.Function("net")
    tq = dict(inp=(0.05, 2), c1=(0.11, -128), c2=(0.21, 5), sc=(0.17, -9), add=(0.3, -128), pool=(0.25, -128), fc=(0.4, 7))
    conv_c = {}
    for name, ci, co, k, in_name in (("c1", cin, c1, 3, "inp"), ("c2", c1, c2, 1, "c1"), ("sc", c1, c2, 1, "c1")):
        w = (rng.standard_normal((co, k, k, ci)) * np.sqrt(2.0 / (k * k * ci))).astype(np.float32)
        b = (rng.standard_normal(co) * 0.05).astype(np.float32)
        conv_c[name] = ops.channelwise_conv_prepare(w, b, tq[in_name][0], ops.SYMMETRIC)
    wf = (rng.standard_normal((classes, c2)) * 0.3).astype(np.float32)
    fq, fs, fo = ops.tensor_rowwise_quantize_i8(wf, ops.ASYMMETRIC)
    fbias_scale = np.float32(tq["pool"][0]) * np.float32(0.01)
    fbias = ops.quantize_bias_i32((rng.standard_normal(classes) * 0.1).astype(np.float32), fbias_scale, 0)

    oh = hw  # 3x3 pad 1
    ph = (oh + 2 - 3) // 2 + 1
    x_in = f.placeholder("input", n * cin * hw * hw * 4)
    result = f.placeholder("result", n * classes * 4)
    a_nhwc = f.activation("nhwc", n * hw * hw * cin * 4)
    a_q = f.activation("q", n * hw * hw * cin)
    a_c1 = f.activation("a_c1", n * oh * oh * c1)
    a_p = f.activation("a_p", n * ph * ph * c1)
    a_c2 = f.activation("a_c2", n * ph * ph * c2)
    a_sc = f.activation("a_sc", n * ph * ph * c2)
    a_add = f.activation("a_add", n * ph * ph * c2)
    a_pool = f.activation("a_pool", n * c2)
    a_fc = f.activation("a_fc", n * classes)

    def conv_syms(name):
        c = conv_c[name]
        return [f.constant(name + "_" + k, c[k]) for k in ("filter", "bias", "filter_scales", "filter_offsets", "bias_scales", "bias_offsets")]

    if quantize_first:
        a_qn = f.activation("q_nchw", n * hw * hw * cin)
        f.quantize(a_qn, x_in, n=n * hw * hw * cin, tqp=tq["inp"])
        f.transpose(a_q, a_qn, dims=(n, cin, hw, hw), shuffle=(0, 2, 3, 1), elem_bytes=1)
    else:
        f.transpose(a_nhwc, x_in, dims=(n, cin, hw, hw), shuffle=(0, 2, 3, 1), elem_bytes=4)
        f.quantize(a_q, a_nhwc, n=n * hw * hw * cin, tqp=tq["inp"])
    s = conv_syms("c1")
    f.channelwise_conv(a_c1, a_q, *s, in_dims=(n, hw, hw, cin), out_dims=(n, oh, oh, c1), kernels=(3, 3), strides=(1, 1),
                       pads=(1, 1, 1, 1), in_tqp=tq["inp"], out_tqp=tq["c1"], act=1)
    f.maxpool(a_p, a_c1, in_dims=(n, oh, oh, c1), out_hw=(ph, ph), kernels=(3, 3), strides=(2, 2), pads=(1, 1), out_offset=tq["c1"][1])
    s = conv_syms("c2")
    f.channelwise_conv(a_c2, a_p, *s, in_dims=(n, ph, ph, c1), out_dims=(n, ph, ph, c2), kernels=(1, 1), strides=(1, 1),
                       pads=(0, 0, 0, 0), in_tqp=tq["c1"], out_tqp=tq["c2"], act=0)
    s = conv_syms("sc")
    f.channelwise_conv(a_sc, a_p, *s, in_dims=(n, ph, ph, c1), out_dims=(n, ph, ph, c2), kernels=(1, 1), strides=(1, 1),
                       pads=(0, 0, 0, 0), in_tqp=tq["c1"], out_tqp=tq["sc"], act=0)
    f.add(a_add, a_c2, a_sc, n=n * ph * ph * c2, lhs_tqp=tq["c2"], rhs_tqp=tq["sc"], dest_tqp=tq["add"])
    f.maxsplat(a_add, a_add, n=n * ph * ph * c2, splat=tq["add"][1])
    f.avgpool(a_pool, a_add, in_dims=(n, ph, ph, c2), out_hw=(1, 1), kernels=(ph, ph), strides=(1, 1), pads=(0, 0),
              in_tqp=tq["add"], out_tqp=tq["pool"])
    f.rowwise_fc(a_fc, a_pool, f.constant("fc_w", fq), f.constant("fc_scales", fs), f.constant("fc_offsets", fo),
                 f.constant("fc_bias", fbias), M=n, K=c2, N=classes, in_tqp=tq["pool"], bias_tqp=(fbias_scale, 0), out_tqp=tq["fc"])
    f.dequantize(result, a_fc, n=n * classes, tqp=tq["fc"])
    f.compile()
    assert f.fused_quantize_transposes == (1 if quantize_first else 0)
    dm.add_network(f)

    x = rng.standard_normal((n, cin, hw, hw)).astype(np.float32)
    out = np.zeros((n, classes), np.float32)
    dm.run_function("net", {"input": x.copy(), "result": out})

    # the same network through the oracle, with parameters derived by the oracle's own restatement
    def oconv(name, t, in_name, out_name, k, pad, act):
        c = conv_c[name]
        pp = oracle.rowwise_requant_params(c["filter_scales"], tq[in_name][0], c["bias_scales"], tq[out_name][0])
        ohw = ops.conv_out_hw(t.shape[1:3], (k, k), (1, 1), (pad,) * 4)
        return oracle.conv2d_i8_i32(t, c["filter"], c["bias"], ohw, (k, k), (1, 1), (pad,) * 4, 1, (1, 1), tq[out_name][1],
                                    tq[in_name][1], c["filter_offsets"], c["bias_offsets"], pp[:3], pp[3:], act, None)

    t = oracle.element_quantize_i8(np.ascontiguousarray(x.transpose(0, 2, 3, 1)), *tq["inp"])
    t = oconv("c1", t, "inp", "c1", 3, 1, 1)
    t = oracle.max_pool_i8(t, (ph, ph), (3, 3), (2, 2), (1, 1, 1, 1), tq["c1"][1])
    y, s_ = oconv("c2", t, "c1", "c2", 1, 0, 0), oconv("sc", t, "c1", "sc", 1, 0, 0)
    lt = oracle.quantize_scale_offset_32to8(np.float32(tq["c2"][0]) / np.float32(tq["add"][0]))
    rt = oracle.quantize_scale_offset_32to8(np.float32(tq["sc"][0]) / np.float32(tq["add"][0]))
    t = oracle.element_maxsplat_i8(oracle.element_add_i8(y, s_, tq["add"][1], tq["c2"][1], tq["sc"][1], lt, rt), tq["add"][1])
    tr = oracle.quantize_scale_offset_32to8(np.float32(tq["add"][0]) / np.float32(tq["pool"][0]) / np.float32(ph * ph))
    t = oracle.avg_pool_i8(t, (1, 1), (ph, ph), (1, 1), (0, 0, 0, 0), True, tq["pool"][1], tq["add"][1], tr)
    pp = oracle.rowwise_requant_params(fs, tq["pool"][0], fbias_scale, tq["fc"][0])
    q = oracle.rowwise_quantized_fc_i8_i32(t.reshape(n, c2), fq, fbias, fo, pp[:3], pp[3:], tq["fc"][1], tq["pool"][1], 0)
    want = oracle.element_dequantize_i8(q, *tq["fc"])
    np.testing.assert_array_equal(out.view(np.uint32), want.view(np.uint32))
    assert len(np.unique(q)) > 5


def test_directions_static_and_resident_placeholders(oracle, dm):
    """Inputs copied in only and outputs out only; a placeholder written once and left on the device
    (a static placeholder); a run on device-resident placeholders fed and read through their device
    addresses (what a peer-to-peer hand-off between partitions uses)."""
    import torch
    table = workloads.fused_table_u8(4000, 64, 9, 0)
    S, cap = 64, 64 * 40
    f = slws_function("drt", table, S, cap)
    dm.add_network(f)
    lengths, idx, w = workloads.bags_poisson(S, 20, 0, 40, 4000, 4, 1)
    want = oracle.frwq_slws_u8_f32(table, w, idx, lengths)
    wp = np.zeros(cap, np.float32); wp[:w.size] = w
    ip = np.zeros(cap, np.int64); ip[:idx.size] = idx
    out = np.full((S, 64), 7.0, np.float32)
    guard_w, guard_i = wp.copy(), ip.copy()
    dm.run_function("drt", {"drt_weights": wp, "drt_indices": ip, "drt_lengths": lengths.copy(), "drt_output": out},
                    outputs={"drt_output"})
    np.testing.assert_allclose(out, want, rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(wp, guard_w)       # inputs are not written back
    np.testing.assert_array_equal(ip, guard_i)
    # static placeholders: weights and indices stay on the device; only lengths travel
    lengths2 = lengths.copy()
    lengths2[::2] = 0
    dm.transfer_static_placeholder("drt", "drt_weights", wp)
    dm.transfer_static_placeholder("drt", "drt_indices", ip)
    out2 = np.zeros((S, 64), np.float32)
    dm.run_function("drt", {"drt_lengths": lengths2, "drt_output": out2}, outputs={"drt_output"})
    np.testing.assert_allclose(out2, oracle.frwq_slws_u8_f32(table, w, idx, lengths2), rtol=1e-5, atol=1e-5)
    # device-resident: write the lengths through the placeholder's device address, run without copies,
    # read the result from its device address
    addr, nbytes = dm.placeholder_address("drt", "drt_lengths")
    assert nbytes == S * 4
    res_addr, res_bytes = dm.placeholder_address("drt", "drt_output")
    assert res_bytes == S * 64 * 4
    def view(address, shape, typestr):
        class Raw:
            pass
        raw = Raw()
        raw.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (address, False), "version": 3}
        return torch.as_tensor(raw, device="cuda")

    view(addr, (S,), "<i4").copy_(torch.from_numpy(lengths).cuda())     # a device-to-device write
    torch.cuda.synchronize()
    dm.run_function_resident("drt")
    res = view(res_addr, (S, 64), "<f4").clone()
    np.testing.assert_allclose(res.cpu().numpy(), want, rtol=1e-5, atol=1e-5)
    with pytest.raises(GlowB200Error):
        dm.placeholder_address("drt", "drt_data")          # a constant, not a placeholder
    with pytest.raises(GlowB200Error):
        dm.run_function_resident("missing")


def test_recommendation_style_network_bit_exact(oracle, dm):
    """A small recommendation model through the runtime, built from the instructions the lowered
    graph holds: Splat (the ones of a lowered SparseLengthsSum) -> fused gather-pool, an fp32
    SparseLengthsSum and a rowwise-quantized one, InsertTensor (lowered Concat) into [B, 3, D],
    Quantize -> per-tensor FullyConnected -> Relu -> Dequantize for the dense features, pairwise dots
    with Quantize fused, Rescale, MatMul, Dequantize.  Checked stage by stage against the oracle."""
    rng = np.random.default_rng(21)
    B, D, rows, cap = 24, 16, 500, 24 * 12
    t8 = workloads.fused_table_u8(rows, D, 3, 0)
    tf = rng.normal(0, 1, (rows, D)).astype(np.float32)
    tq8 = rng.integers(0, 256, (rows, D), dtype=np.uint8)
    sc8, of8 = rng.uniform(0.001, 0.01, rows).astype(np.float32), rng.uniform(-1, 1, rows).astype(np.float32)
    lengths, idx, w = workloads.bags_poisson(B, 6, 0, 12, rows, 8, 1)
    n = int(lengths.sum())
    din = 20
    wfc = rng.integers(-127, 128, (din, D)).astype(np.int8)          # [K, N]
    bfc = rng.integers(-500, 500, D).astype(np.int32)
    tq = dict(x=(0.04, 3), w=(0.01, 0), b=(0.0004, 0), h=(0.08, -20), r=(0.08, -128), inter=(0.9, -10), rs=(1.3, 4),
              m=(0.02, 1), mm=(2.5, -3))
    wm = rng.integers(-127, 128, (D + 6, 5)).astype(np.int8)          # MatMul right-hand side [K, N]
    width = D + 4 * 3 // 2

    f = runtime.Function("rec")
    c8, cf, cq = f.constant("t8", t8), f.constant("tf", tf), f.constant("tq8", tq8)
    csc, cof = f.constant("sc8", sc8), f.constant("of8", of8)
    p_idx, p_len, p_w = f.placeholder("idx", cap * 8), f.placeholder("len", B * 4), f.placeholder("w", cap * 4)
    p_x, p_out = f.placeholder("x", B * din * 4), f.placeholder("out", B * 5 * 4)
    p_pooled = f.placeholder("pooled", B * 3 * D * 4)                  # kept as a placeholder so the test can read it
    a_ones, a_e0, a_e1, a_e2 = (f.activation(k, s) for k, s in (("ones", cap * 4), ("e0", B * D * 4), ("e1", B * D * 4), ("e2", B * D * 4)))
    a_xq, a_h, a_hr, a_hf = f.activation("xq", B * din), f.activation("h", B * D), f.activation("hr", B * D), f.activation("hf", B * D * 4)
    a_i, a_ir, a_m = f.activation("inter", B * width), f.activation("inter_r", B * width), f.activation("m", B * 5)
    f.splat(a_ones, n=cap, value=1.0)
    f.frwq_slws(a_e0, c8, a_ones, p_idx, p_len, kind=ops.UINT8_FUSED, rows=rows, in_line=D + 8, out_line=D, segments=B, num_indices=cap)
    f.sparse_lengths_sum(a_e1, cf, None, p_idx, p_len, rows=rows, line=D, segments=B, num_indices=cap)
    f.rowwise_quantized_slws(a_e2, cq, csc, cof, p_w, p_idx, p_len, rows=rows, line=D, segments=B, num_indices=cap)
    for j, a in enumerate((a_e0, a_e1, a_e2)):
        f.insert_tensor(p_pooled, a, rows=B, width_bytes=D * 4, dest_pitch_bytes=3 * D * 4, dest_offset_bytes=j * D * 4)
    f.quantize(a_xq, p_x, n=B * din, tqp=tq["x"])
    f.fully_connected(a_h, a_xq, f.constant("wfc", wfc), f.constant("bfc", bfc), M=B, K=din, N=D, in_tqp=tq["x"], w_tqp=tq["w"],
                      bias_tqp=tq["b"], out_tqp=tq["h"])
    f.relu(a_hr, a_h, n=B * D, src_tqp=tq["h"], dest_tqp=tq["r"])
    f.dequantize(a_hf, a_hr, n=B * D, tqp=tq["r"])
    f.pairwise_dot(a_i, a_hf, p_pooled, batch=B, tables=3, dim=D, quant=tq["inter"])
    f.rescale(a_ir, a_i, n=B * width, in_tqp=tq["inter"], out_tqp=tq["rs"])
    f.matmul(a_m, a_ir, f.constant("wm", wm), M=B, K=width, N=5, lhs_tqp=tq["rs"], rhs_tqp=tq["m"], out_tqp=tq["mm"])
    f.dequantize(p_out, a_m, n=B * 5, tqp=tq["mm"])
    f.compile()
    dm.add_network(f)

    x = rng.normal(0, 1, (B, din)).astype(np.float32)
    ip = np.zeros(cap, np.int64); ip[:n] = idx
    wp = np.zeros(cap, np.float32); wp[:n] = w
    out, pooled = np.zeros((B, 5), np.float32), np.zeros((B, 3, D), np.float32)
    dm.run_function("rec", {"idx": ip, "len": lengths.copy(), "w": wp, "x": x.copy(), "out": out, "pooled": pooled},
                    outputs={"out", "pooled"})

    e0 = oracle.frwq_slws_u8_f32(t8, np.ones(n, np.float32), idx, lengths)
    e1 = oracle.sparse_lengths_sum_f32(tf, idx, lengths)
    e2 = oracle.rowwise_quantized_slws_f32(tq8, sc8, of8, w, idx, lengths)
    np.testing.assert_allclose(pooled[:, 0], e0, rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(pooled[:, 1].view(np.uint32), e1.view(np.uint32))
    np.testing.assert_array_equal(pooled[:, 2].view(np.uint32), e2.view(np.uint32))
    # the dense part from the pooled vectors the device produced: bit for bit
    q = oracle.quantize_scale_offset_32to8
    xq = oracle.element_quantize_i8(x, *tq["x"])
    mm = np.float32(tq["x"][0]) * np.float32(tq["w"][0])
    h = oracle.fc_i8_i32(xq, wfc, bfc, tq["h"][1], tq["x"][1], tq["w"][1], tq["b"][1], q(np.float32(tq["b"][0]) / mm),
                         q(mm / np.float32(tq["h"][0])))
    hr = oracle.element_relu_i8(h, tq["h"][1], tq["r"][1], q(np.float32(tq["h"][0]) / np.float32(tq["r"][0])))
    hf = oracle.element_dequantize_i8(hr, *tq["r"])
    inter = oracle.element_quantize_i8(oracle.pairwise_dot_interaction(hf, pooled), *tq["inter"])
    ir = oracle.element_rescale_i8(inter, tq["rs"][1], tq["inter"][1], q(np.float32(tq["inter"][0]) / np.float32(tq["rs"][0])))
    m = oracle.matmul_i8(ir, wm, tq["mm"][1], tq["rs"][1], tq["m"][1],
                         q(np.float32(tq["rs"][0]) * np.float32(tq["m"][0]) / np.float32(tq["mm"][0])))
    want = oracle.element_dequantize_i8(m, *tq["mm"])
    np.testing.assert_array_equal(out.view(np.uint32), want.view(np.uint32))
    assert len(np.unique(m)) > 5


def test_split_embedding_and_dynamic_fc_instructions(oracle, dm):
    """A table-batched embedding layer feeding a dynamically quantized FC, as one loaded function:
    IntNBitSplitEmbeddingBags (fp16 result) -> DynamicRowwiseQuantizedFullyConnected."""
    rng = np.random.default_rng(91)
    specs = [(ops.EST_INT4, 32, 400), (ops.EST_INT8, 16, 300), (ops.EST_FLOAT16, 16, 200)]
    B, N = 24, 40
    chunks, offs, at = [], [], 0
    for ty, d, rows in specs:
        rb = ops.split_embedding_row_bytes(d, ty)
        tab = rng.integers(0, 256, (rows, rb), dtype=np.uint8)
        if ty == ops.EST_FLOAT16:
            tab[:, :2 * d] = rng.normal(0, 1, (rows, d)).astype(np.float16).view(np.uint8)
        else:
            hdr = np.stack([rng.uniform(0.001, 0.02, rows), rng.uniform(-1, 1, rows)], 1).astype(np.float16)
            tab[:, :4] = hdr.view(np.uint8)
        offs.append(at)
        chunks.append(tab.reshape(-1))
        at += tab.size
    weights = np.concatenate(chunks + [np.zeros(16, np.uint8)])
    T = len(specs)
    dims = np.array([0] + [d for _, d, _ in specs]).cumsum().astype(np.int32)
    D = int(dims[-1])
    lens = rng.poisson(5, (T, B))
    offsets = np.concatenate([[0], np.cumsum(lens.reshape(-1))]).astype(np.int32)
    idx = np.concatenate([rng.integers(0, rows, int(lens[i].sum())) for i, (_, _, rows) in enumerate(specs)]).astype(np.int32)
    max_idx = idx.size + 7
    w = rng.integers(-128, 128, (D, N), dtype=np.int8)
    bias = rng.normal(0, 1, N).astype(np.float32)
    scales = rng.uniform(0.001, 0.02, N).astype(np.float32)
    woff = rng.integers(-5, 5, N).astype(np.int32)

    f = runtime.Function("tbe_dynfc")
    cw = f.constant("weights", weights)
    cpl = f.constant("placements", np.full(T, ops.PLACEMENT_HOST, np.int32))
    cwo = f.constant("weights_offsets", np.array(offs, np.int32))
    cty = f.constant("weights_tys", np.array([s[0] for s in specs], np.uint8))
    cdo = f.constant("dim_offsets", dims)
    pidx = f.placeholder("indices", max_idx * 4)
    poff = f.placeholder("offsets", offsets.size * 4)
    pooled = f.activation("pooled", B * D * 2)
    cfw = f.constant("fc_weights", w)
    cfb = f.constant("fc_bias", bias)
    cfs = f.constant("fc_scales", scales)
    cfo = f.constant("fc_offsets", woff)
    out = f.placeholder("out", B * N * 2)
    f.split_embedding_bags(pooled, cw, cw, cpl, cwo, cty, cdo, pidx, poff, dev_bytes=weights.size, uvm_bytes=weights.size,
                           num_tables=T, total_dims=D, num_indices=max_idx, bags_per_table=B, out_fp16=True)
    f.dynamic_quantized_fc(out, pooled, cfw, cfb, cfs, cfo, M=B, K=D, N=N)
    f.compile()
    dm.add_network(f)
    ip = np.zeros(max_idx, np.int32); ip[:idx.size] = idx
    got = np.zeros((B, N), np.float16)
    dm.run_function("tbe_dynfc", {"indices": ip, "offsets": offsets, "out": got})
    want_pooled = oracle.int_nbit_split_embedding_bags(weights, weights, np.full(T, 3, np.int32), np.array(offs, np.int32),
                                                       np.array([s[0] for s in specs], np.uint8), dims, D, idx, offsets,
                                                       out_fp16=True)
    want = oracle.dynamic_rowwise_quantized_fc(want_pooled, w, bias, scales, woff)
    np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))


def test_arithmetic_glue_instructions(oracle, dm):
    """Sub, Max, Mul, Div and BatchedAdd as instructions: the runtime derives their integer
    parameters from the tensors' scales as LLVMIRGen does; results against the oracle."""
    rng = np.random.default_rng(17)
    n, rows = 4096, 64
    a = rng.integers(-128, 128, n).astype(np.int8)
    b = rng.integers(-128, 128, n).astype(np.int8)
    sl = rng.integers(-128, 128, n // rows).astype(np.int8)
    ta, tb, td, ts = (0.02, -3), (0.05, 9), (0.04, 5), (0.03, 1)
    f = runtime.Function("arith")
    pa, pb, psl = f.placeholder("a", n), f.placeholder("b", n), f.placeholder("slice", n // rows)
    outs = {k: f.placeholder(k, n) for k in ("sub", "max", "mul", "div", "badd")}
    f.binary(ops.BINARY_SUB, outs["sub"], pa, pb, n=n, lhs_tqp=ta, rhs_tqp=tb, dest_tqp=td)
    f.binary(ops.BINARY_MAX, outs["max"], pa, pb, n=n, lhs_tqp=ta, rhs_tqp=tb, dest_tqp=td)
    f.muldiv(False, outs["mul"], pa, pb, n=n, lhs_tqp=ta, rhs_tqp=tb, dest_tqp=td)
    f.muldiv(True, outs["div"], pa, pb, n=n, lhs_tqp=ta, rhs_tqp=tb, dest_tqp=td)
    f.batched_add(outs["badd"], pa, psl, num_slices=rows, slice_size=n // rows, batch_tqp=ta, slice_tqp=ts, dest_tqp=td)
    f.compile()
    dm.add_network(f)
    got = {k: np.zeros(n, np.int8) for k in outs}
    dm.run_function("arith", dict(a=a, b=b, slice=sl, **got))
    q = oracle.quantize_scale_offset_32to8
    f32 = np.float32
    lt, rt = q(f32(ta[0]) / f32(td[0])), q(f32(tb[0]) / f32(td[0]))
    np.testing.assert_array_equal(got["sub"], oracle.element_binary_i8(1, a, b, td[1], ta[1], tb[1], lt, rt))
    np.testing.assert_array_equal(got["max"], oracle.element_binary_i8(2, a, b, td[1], ta[1], tb[1], lt, rt))
    np.testing.assert_array_equal(got["mul"], oracle.element_muldiv_i8(False, a, b, td[1], ta[1], tb[1],
                                                                     q(f32(ta[0]) * f32(tb[0]) / f32(td[0]))))
    np.testing.assert_array_equal(got["div"], oracle.element_muldiv_i8(True, a, b, td[1], ta[1], tb[1],
                                                                     q(f32(ta[0]) / (f32(tb[0]) * f32(td[0])))))
    np.testing.assert_array_equal(got["badd"], oracle.batched_add_i8(a.reshape(rows, -1), sl, td[1], ta[1], ts[1], lt,
                                                                      q(f32(ts[0]) / f32(td[0]))).reshape(-1))


def _pooling_network(name, tables, B, max_n, idx_dtype=np.int32, static=True):
    """T FRWQ-SLWS nodes over T tables whose indices, weights and lengths are views of three
    shared placeholders ([T, max_n] indices and weights, [T, B] lengths) and whose results are
    the T row blocks of one [T, B, D] output -- the per-table SparseLengthsSum nodes of a
    recommendation model with its inputs in one arena."""
    T = len(tables)
    rows, in_line = tables[0].shape
    D = in_line - 8
    isz = np.dtype(idx_dtype).itemsize
    f = runtime.Function(name)
    tabs = [(f.static_placeholder if static else f.placeholder)("%s_table%d" % (name, t), tables[t].nbytes) for t in range(T)]
    idx = f.placeholder(name + "_indices", T * max_n * isz)
    w = f.placeholder(name + "_weights", T * max_n * 4)
    ln = f.placeholder(name + "_lengths", T * B * 4)
    out = f.placeholder(name + "_output", T * B * D * 4)
    for t in range(T):
        f.frwq_slws((out, t * B * D * 4), tabs[t], (w, t * max_n * 4), (idx, t * max_n * isz), (ln, t * B * 4),
                    kind=ops.UINT8_FUSED, rows=rows, in_line=in_line, out_line=D, segments=B, num_indices=max_n,
                    idx64=isz == 8)
    return f.compile()


def _pooling_request(dm, T, B, max_n, rows, seed, idx_dtype=np.int32):
    idx = dm.io_buffer((T, max_n), idx_dtype)
    w = dm.io_buffer((T, max_n), np.float32)
    ln = dm.io_buffer((T, B), np.int32)
    idx[:], w[:] = 0, 0
    per_table = []
    for t in range(T):
        l, i, ww = workloads.bags_poisson(B, 12, 0, 30, rows, seed, t)
        assert i.size <= max_n
        ln[t], idx[t, :i.size], w[t, :i.size] = l, i, ww
        per_table.append((l, i, ww))
    return idx, w, ln, per_table


def test_views_batched_pooling_and_asynchronous_requests(oracle, dm):
    """Operands that are views of larger tensors; consecutive pooling nodes fused into one batched
    launch; int32 indices; static tables shared by two execution contexts; four requests through
    the asynchronous call with two in flight -- every result against the oracle."""
    T, B, rows, D, max_n = 6, 64, 4000, 64, 64 * 30
    tables = [workloads.fused_table_u8(rows, D, 90, t) for t in range(T)]
    f = _pooling_network("pool", tables, B, max_n)
    assert f.batched_pooling_launches == 1
    dm.set_context_count(2)
    dm.add_network(f)
    for t in range(T):
        dm.transfer_static_placeholder("pool", "pool_table%d" % t, tables[t])
    reqs = [_pooling_request(dm, T, B, max_n, rows, 200 + r) for r in range(4)]
    outs = [dm.io_buffer((T, B, D), np.float32) for _ in range(4)]
    tickets = []
    for r in range(4):
        idx, w, ln, _ = reqs[r]
        outs[r][:] = np.nan
        tickets.append(dm.run_function_async("pool", {"pool_indices": idx, "pool_weights": w, "pool_lengths": ln,
                                                      "pool_output": outs[r]}, outputs=("pool_output",)))
        if r >= 1:
            dm.wait(tickets[r - 1])  # two requests in flight at most, as a serving loop keeps them
    dm.wait(tickets[-1])
    for r in range(4):
        for t in range(T):
            l, i, ww = reqs[r][3][t]
            want = oracle.frwq_slws_u8_f32(tables[t], ww, i.astype(np.int64), l)
            np.testing.assert_allclose(outs[r][t], want, rtol=1e-5, atol=1e-5)
    # the synchronous call on the same network gives the same bits
    idx, w, ln, _ = reqs[0]
    again = np.zeros((T, B, D), np.float32)
    dm.run_function("pool", {"pool_indices": idx, "pool_weights": w, "pool_lengths": ln, "pool_output": again},
                    outputs=("pool_output",))
    np.testing.assert_array_equal(again, outs[0])
    # a bad index surfaces from wait(), and the next request is clean
    idx2 = idx.copy()
    idx2[3, 0] = rows + 5
    t_bad = dm.run_function_async("pool", {"pool_indices": idx2, "pool_weights": w, "pool_lengths": ln,
                                           "pool_output": again}, outputs=("pool_output",))
    t_ok = dm.run_function_async("pool", {"pool_indices": idx, "pool_weights": w, "pool_lengths": ln,
                                          "pool_output": outs[1]}, outputs=("pool_output",))
    with pytest.raises(GlowB200Error, match="invalid sparse input"):
        dm.wait(t_bad)
    dm.wait(t_ok)
    np.testing.assert_array_equal(outs[1], outs[0])


def test_batched_pooling_equals_single_launches(oracle, dm):
    """The same network with its pooling nodes kept apart (a Copy between them breaks the run)
    gives the same bits as the fused launch."""
    T, B, rows, D, max_n = 4, 40, 3000, 128, 40 * 30
    tables = [workloads.fused_table_u8(rows, D, 95, t) for t in range(T)]
    fused = _pooling_network("fusedp", tables, B, max_n, np.int64, static=False)
    apart = runtime.Function("apartp")
    isz = 8
    tabs = [apart.placeholder("apartp_table%d" % t, tables[t].nbytes) for t in range(T)]
    idx = apart.placeholder("apartp_indices", T * max_n * isz)
    w = apart.placeholder("apartp_weights", T * max_n * 4)
    ln = apart.placeholder("apartp_lengths", T * B * 4)
    out = apart.placeholder("apartp_output", T * B * D * 4)
    scratch = apart.activation("apartp_scratch", 64)
    for t in range(T):
        apart.frwq_slws((out, t * B * D * 4), tabs[t], (w, t * max_n * 4), (idx, t * max_n * isz), (ln, t * B * 4),
                        kind=ops.UINT8_FUSED, rows=rows, in_line=D + 8, out_line=D, segments=B, num_indices=max_n)
        apart.copy(scratch, scratch, nbytes=64)
    apart.compile()
    assert fused.batched_pooling_launches == 1 and apart.batched_pooling_launches == 0
    dm.add_network(fused)
    dm.add_network(apart)
    idxh, wh, lnh, per = _pooling_request(dm, T, B, max_n, rows, 300, np.int64)
    res = {}
    for name in ("fusedp", "apartp"):
        o = np.zeros((T, B, D), np.float32)
        b = {name + "_indices": idxh, name + "_weights": wh, name + "_lengths": lnh, name + "_output": o}
        b.update({"%s_table%d" % (name, t): tables[t] for t in range(T)})
        dm.run_function(name, b, outputs=(name + "_output",))
        res[name] = o
    np.testing.assert_array_equal(res["fusedp"], res["apartp"])
    for t in range(T):
        l, i, ww = per[t]
        np.testing.assert_allclose(res["fusedp"][t], oracle.frwq_slws_u8_f32(tables[t], ww, i, l), rtol=1e-5, atol=1e-5)
