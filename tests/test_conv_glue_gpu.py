"""Int8 convolution and glue operators against the CPU oracle: bit-exact."""
import numpy as np
import pytest
import torch

from glow_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


CONV_CASES = [
    # n, ih, iw, ic, oc, kernel, stride, pads, group, dilation, act
    (2, 14, 14, 64, 64, (3, 3), (1, 1), (1, 1, 1, 1), 1, (1, 1), 1),     # ResNet 3x3
    (2, 14, 14, 64, 256, (1, 1), (1, 1), (0, 0, 0, 0), 1, (1, 1), 0),    # pointwise: no im2col
    (2, 14, 14, 128, 256, (1, 1), (2, 2), (0, 0, 0, 0), 1, (1, 1), 0),   # strided shortcut
    (1, 30, 30, 3, 64, (7, 7), (2, 2), (3, 3, 3, 3), 1, (1, 1), 1),      # stem: K = 147 -> padded to 160
    (3, 9, 11, 32, 48, (3, 3), (2, 2), (1, 1, 1, 1), 1, (1, 1), 2),      # clip
    (1, 11, 11, 16, 24, (3, 3), (1, 1), (2, 2, 2, 2), 1, (2, 2), 5),     # dilation, leaky relu
    (1, 12, 10, 6, 8, (3, 3), (2, 2), (1, 1, 1, 1), 2, (1, 1), 1),       # groups -> direct kernel
    (1, 5, 5, 8, 8, (3, 3), (1, 1), (1, 1, 1, 1), 8, (1, 1), 0),         # depthwise
    (2, 7, 7, 20, 10, (1, 1), (1, 1), (0, 0, 0, 0), 1, (1, 1), 0),       # C not a multiple of 16
    (2, 64, 48, 3, 32, (7, 7), (2, 2), (3, 3, 3, 3), 1, (1, 1), 1),      # stem shape: rows staged in shared memory
    (1, 17, 13, 5, 12, (3, 5), (1, 2), (1, 2, 1, 2), 1, (1, 1), 0),      # odd channel count, rectangular window
    (1, 12, 12, 12, 16, (3, 3), (1, 1), (2, 2, 2, 2), 1, (2, 2), 0),     # dilation with C not a multiple of 16
    # stride-1 windows over 64 / 128k channels with symmetric filters: the shifted-rows path (no im2col)
    (2, 9, 13, 128, 96, (3, 3), (1, 1), (1, 1, 1, 1), 1, (1, 1), 1),
    (1, 10, 7, 256, 300, (3, 3), (1, 1), (1, 1, 1, 1), 1, (1, 1), 0),
    (3, 8, 8, 64, 64, (5, 5), (1, 1), (2, 2, 2, 2), 1, (1, 1), 1),       # 5 taps per row: an odd tap without partner
    (2, 11, 6, 64, 40, (2, 2), (1, 1), (0, 0, 0, 0), 1, (1, 1), 0),      # even window, no padding
    (1, 6, 9, 128, 32, (1, 3), (1, 1), (0, 1, 0, 1), 1, (1, 1), 2),      # one-row window, clip
    (2, 7, 7, 64, 16, (3, 3), (1, 1), (2, 0, 1, 2), 1, (1, 1), 0),       # unequal pads
    # stride-2 windows over 128k channels with symmetric filters: shifted rows over four parity planes
    (2, 9, 11, 128, 48, (3, 3), (2, 2), (1, 1, 1, 1), 1, (1, 1), 1),
    (1, 12, 10, 256, 40, (3, 3), (2, 2), (1, 1, 1, 1), 1, (1, 1), 0),
    (2, 8, 8, 128, 32, (5, 5), (2, 2), (2, 2, 2, 2), 1, (1, 1), 2),
    (1, 9, 9, 128, 16, (3, 3), (2, 2), (0, 1, 1, 0), 1, (1, 1), 0),      # unequal pads
    (1, 10, 10, 128, 24, (2, 2), (2, 2), (0, 0, 0, 0), 1, (1, 1), 0),    # window = stride
]


def _conv_inputs(oracle, case, symmetric):
    n, ih, iw, ic, oc, k, s, p, g, d, act = case
    rng = np.random.default_rng(ic * 1000 + oc * 7 + k[0])
    K = k[0] * k[1] * ic // g
    c = dict(
        inp=rng.integers(-128, 128, (n, ih, iw, ic)).astype(np.int8),
        filt=rng.integers(-127, 128, (oc, k[0], k[1], ic // g)).astype(np.int8),
        bias=rng.integers(-3000, 3000, oc).astype(np.int32),
        fo=np.zeros(oc, np.int32) if symmetric else rng.integers(-3, 4, oc).astype(np.int32),
        bo=np.zeros(oc, np.int32) if symmetric else rng.integers(-5, 5, oc).astype(np.int32))
    fs = rng.uniform(0.002, 0.02, oc).astype(np.float32)
    in_scale = np.float32(0.04)
    out_scale = np.float32(0.9 * np.sqrt(K / 72.0))
    c["pp"] = oracle.rowwise_requant_params(fs, in_scale, in_scale * fs, out_scale)
    c["act_args"] = {2: [-20, 60], 5: list(oracle.quantize_scale_offset_32to8(0.1))}.get(act)
    return c


@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("symmetric", [True, False])
def test_channelwise_conv_bit_exact(oracle, case, symmetric):
    n, ih, iw, ic, oc, k, s, p, g, d, act = case
    c = _conv_inputs(oracle, case, symmetric)
    ohw = ops.conv_out_hw((ih, iw), k, s, p, d)
    want = oracle.conv2d_i8_i32(c["inp"], c["filt"], c["bias"], ohw, k, s, p, g, d, 4, -2, c["fo"], c["bo"], c["pp"][:3],
                                c["pp"][3:], act, c["act_args"])
    pp = [t(a) for a in c["pp"]]
    st = ops.new_status(DEV)
    for flags in (ops.FC_WEIGHT_OFFSETS_ZERO if symmetric else 0, ops.FC_FORCE_ANY_SHAPE_KERNEL):
        got = ops.channelwise_quantized_conv2d(t(c["inp"]), t(c["filt"]), t(c["bias"]), k, s, p, g, d, 4, -2, t(c["fo"]),
                                               t(c["bo"]), pp[:3], pp[3:], act, c["act_args"], flags=flags, status=st)
        np.testing.assert_array_equal(got.cpu().numpy(), want)
    assert int(st.item()) == 0
    assert len(np.unique(want)) > 10


@pytest.mark.parametrize("case", [CONV_CASES[0], CONV_CASES[3], CONV_CASES[6]])
def test_per_tensor_conv_bit_exact(oracle, case):
    n, ih, iw, ic, oc, k, s, p, g, d, act = case
    c = _conv_inputs(oracle, case, False)
    ohw = ops.conv_out_hw((ih, iw), k, s, p, d)
    bt = [int(x[0]) for x in c["pp"][:3]]
    ot = [int(x[0]) for x in c["pp"][3:]]
    want = oracle.conv2d_i8_i32(c["inp"], c["filt"], c["bias"], ohw, k, s, p, g, d, 4, -2, c["fo"][:1], c["bo"][:1], bt, ot,
                                act, c["act_args"], per_channel=False)
    got = ops.conv2d_i8(t(c["inp"]), t(c["filt"]), t(c["bias"]), k, s, p, g, d, 4, -2, int(c["fo"][0]), int(c["bo"][0]),
                        bt, ot, act, c["act_args"])
    np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_resnet_sized_conv_against_direct_kernel():
    """A ResNet-50 layer at batch 64 (3x3, 128 channels, 28x28): the tensor-core path against the
    direct kernel on the device (the CPU oracle covers the smaller cases above)."""
    rng = np.random.default_rng(5)
    n, hw, ch = 64, 28, 128
    inp = t(rng.integers(-128, 128, (n, hw, hw, ch)).astype(np.int8))
    filt = t(rng.integers(-127, 128, (ch, 3, 3, ch)).astype(np.int8))
    bias = t(rng.integers(-3000, 3000, ch).astype(np.int32))
    zeros = torch.zeros(ch, dtype=torch.int32, device=DEV)
    fs = rng.uniform(0.002, 0.02, ch).astype(np.float32)
    pp = [t(a) for a in ops.rowwise_requant_params(fs, 0.04, np.float32(0.04) * fs, np.float32(3.5))]
    args = (inp, filt, bias, (3, 3), (1, 1), (1, 1, 1, 1), 1, (1, 1), 3, -5, zeros, zeros, pp[:3], pp[3:], 1, None)
    a = ops.channelwise_quantized_conv2d(*args, flags=ops.FC_WEIGHT_OFFSETS_ZERO)
    b = ops.channelwise_quantized_conv2d(*args, flags=ops.FC_FORCE_ANY_SHAPE_KERNEL)
    assert torch.equal(a, b)
    assert a.unique().numel() > 50


def test_elementwise_and_pools_bit_exact(oracle):
    rng = np.random.default_rng(13)
    a = rng.integers(-128, 128, 100_003).astype(np.int8)
    b = rng.integers(-128, 128, 100_003).astype(np.int8)
    lt = ops.quantize_scale_offset_32to8(0.7)
    rt = ops.quantize_scale_offset_32to8(1.9)
    np.testing.assert_array_equal(ops.element_add_i8(t(a), t(b), 5, -3, 9, lt, rt).cpu().numpy(),
                                  oracle.element_add_i8(a, b, 5, -3, 9, lt, rt))
    np.testing.assert_array_equal(ops.element_add_maxsplat_i8(t(a), t(b), 5, -3, 9, lt, rt, -20).cpu().numpy(),
                                  oracle.element_maxsplat_i8(oracle.element_add_i8(a, b, 5, -3, 9, lt, rt), -20))
    np.testing.assert_array_equal(ops.element_relu_i8(t(a), -10, 4, lt).cpu().numpy(), oracle.element_relu_i8(a, -10, 4, lt))
    np.testing.assert_array_equal(ops.element_maxsplat_i8(t(a), -7).cpu().numpy(), oracle.element_maxsplat_i8(a, -7))
    np.testing.assert_array_equal(ops.element_rescale_i8(t(a), 3, -2, rt).cpu().numpy(), oracle.element_rescale_i8(a, 3, -2, rt))
    f = (rng.standard_normal(50_000) * 3).astype(np.float32)
    f[:8] = [0.5 * 0.05, 1.5 * 0.05, 2.5 * 0.05, -0.5 * 0.05, -1.5 * 0.05, 1000.0, -1000.0, 0.0]
    np.testing.assert_array_equal(ops.element_quantize_i8(t(f), 0.05, 3).cpu().numpy(), oracle.element_quantize_i8(f, 0.05, 3))
    np.testing.assert_array_equal(ops.element_dequantize_i8(t(a), 0.037, -4).cpu().numpy().view(np.uint32),
                                  oracle.element_dequantize_i8(a, 0.037, -4).view(np.uint32))
    x = rng.integers(-128, 128, (2, 23, 19, 24)).astype(np.int8)
    for k, s, p in [((3, 3), (2, 2), (1, 1, 1, 1)), ((2, 2), (2, 2), (0, 0, 0, 0)), ((7, 7), (1, 1), (3, 3, 3, 3)),
                    ((23, 19), (1, 1), (0, 0, 0, 0))]:
        ohw = ops.conv_out_hw((23, 19), k, s, p)
        np.testing.assert_array_equal(ops.max_pool_i8(t(x), k, s, p, -7).cpu().numpy(), oracle.max_pool_i8(x, ohw, k, s, p, -7))
        for cip in (True, False):
            area = np.float32(k[0] * k[1]) if cip else np.float32(1)
            tr = ops.quantize_scale_offset_32to8(np.float32(0.03) / np.float32(0.05) / area)
            np.testing.assert_array_equal(ops.avg_pool_i8(t(x), k, s, p, cip, 3, -4, tr).cpu().numpy(),
                                          oracle.avg_pool_i8(x, ohw, k, s, p, cip, 3, -4, tr))


def test_elementwise_kernels_on_unaligned_tensors(oracle):
    """Tensors that do not start on 16-byte boundaries take the element-at-a-time path of the
    element-wise kernels: same results."""
    rng = np.random.default_rng(17)
    a = rng.integers(-128, 128, 5_001).astype(np.int8)
    b = rng.integers(-128, 128, 5_001).astype(np.int8)
    lt, rt = ops.quantize_scale_offset_32to8(0.7), ops.quantize_scale_offset_32to8(1.9)
    da, dl, dr = t(a)[1:], t(a)[1:4_999], t(b)[3:5_001]
    assert da.data_ptr() % 16 and dr.data_ptr() % 16 and dl.numel() == dr.numel()
    np.testing.assert_array_equal(ops.element_add_maxsplat_i8(dl, dr, 5, -3, 9, lt, rt, -20).cpu().numpy(),
                                  oracle.element_maxsplat_i8(oracle.element_add_i8(a[1:4_999], b[3:5_001], 5, -3, 9, lt, rt), -20))
    np.testing.assert_array_equal(ops.element_relu_i8(da, -10, 4, lt).cpu().numpy(), oracle.element_relu_i8(a[1:], -10, 4, lt))
    np.testing.assert_array_equal(ops.element_rescale_i8(da, 3, -2, rt).cpu().numpy(), oracle.element_rescale_i8(a[1:], 3, -2, rt))
    f = (rng.standard_normal(1_003) * 3).astype(np.float32)
    np.testing.assert_array_equal(ops.element_quantize_i8(t(f)[1:], 0.05, 3).cpu().numpy(), oracle.element_quantize_i8(f[1:], 0.05, 3))
    np.testing.assert_array_equal(ops.element_dequantize_i8(da, 0.037, -4).cpu().numpy().view(np.uint32),
                                  oracle.element_dequantize_i8(a[1:], 0.037, -4).view(np.uint32))


def test_max_pool_sixteen_channels_per_thread(oracle):
    rng = np.random.default_rng(29)
    x = rng.integers(-128, 128, (3, 21, 18, 64)).astype(np.int8)
    for k, s, p in [((3, 3), (2, 2), (1, 1, 1, 1)), ((2, 2), (2, 2), (0, 0, 0, 0)), ((5, 5), (3, 3), (2, 2, 2, 2))]:
        ohw = ops.conv_out_hw((21, 18), k, s, p)
        np.testing.assert_array_equal(ops.max_pool_i8(t(x), k, s, p, -7).cpu().numpy(), oracle.max_pool_i8(x, ohw, k, s, p, -7))


def test_transpose():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 5, 7, 11)).astype(np.float32)
    for sh in [(0, 2, 3, 1), (0, 3, 1, 2), (3, 2, 1, 0)]:
        np.testing.assert_array_equal(ops.transpose(t(x), sh).cpu().numpy(), np.transpose(x, sh))
    y = rng.integers(-128, 128, (6, 9, 4)).astype(np.int8)
    np.testing.assert_array_equal(ops.transpose(t(y), (2, 0, 1)).cpu().numpy(), np.transpose(y, (2, 0, 1)))
    q = rng.integers(-128, 128, (2, 3, 10, 12)).astype(np.int8)   # NCHW -> NHWC with few channels
    np.testing.assert_array_equal(ops.transpose(t(q), (0, 2, 3, 1)).cpu().numpy(), np.transpose(q, (0, 2, 3, 1)))
    # Quantize + Transpose in one pass == the two kernels one after the other
    f = (rng.standard_normal((2, 3, 10, 12)) * 3).astype(np.float32)
    for sh in [(0, 2, 3, 1), (0, 3, 1, 2), (3, 2, 1, 0)]:
        two = ops.transpose(ops.element_quantize_i8(t(f), 0.037, -5), sh)
        assert torch.equal(ops.quantize_transpose_i8(t(f), sh, 0.037, -5), two)
    z = rng.integers(-128, 128, (40, 33)).astype(np.int8)
    np.testing.assert_array_equal(ops.transpose(t(z), (1, 0)).cpu().numpy(), z.T)


def test_binary_muldiv_batched_add_bit_exact(oracle):
    """Sub / Max / Min, Mul / Div and BatchedAdd (int8 and int32 slice) against the oracle."""
    rng = np.random.default_rng(29)
    a = rng.integers(-128, 128, 70_001).astype(np.int8)
    b = rng.integers(-128, 128, 70_001).astype(np.int8)
    lt, rt = ops.quantize_scale_offset_32to8(0.7), ops.quantize_scale_offset_32to8(1.9)
    for op in (ops.BINARY_ADD, ops.BINARY_SUB, ops.BINARY_MAX, ops.BINARY_MIN):
        np.testing.assert_array_equal(ops.element_binary_i8(op, t(a), t(b), 5, -3, 9, lt, rt).cpu().numpy(),
                                      oracle.element_binary_i8(op, a, b, 5, -3, 9, lt, rt))
    tm, td = ops.quantize_scale_offset_32to8(0.011), ops.quantize_scale_offset_32to8(3.3)
    np.testing.assert_array_equal(ops.element_muldiv_i8(False, t(a), t(b), 2, -3, 9, tm).cpu().numpy(),
                                  oracle.element_muldiv_i8(False, a, b, 2, -3, 9, tm))
    np.testing.assert_array_equal(ops.element_muldiv_i8(True, t(a), t(b), 2, -3, 9, td).cpu().numpy(),
                                  oracle.element_muldiv_i8(True, a, b, 2, -3, 9, td))      # zero divisors included
    batch = rng.integers(-128, 128, (333, 517)).astype(np.int8)
    for sl in (rng.integers(-128, 128, 517).astype(np.int8), rng.integers(-100000, 100000, 517).astype(np.int32)):
        st = ops.quantize_scale_offset_32to8(0.004 if sl.dtype == np.int32 else 1.3)
        np.testing.assert_array_equal(ops.batched_add_i8(t(batch), t(sl), -6, 4, 1, lt, st).cpu().numpy(),
                                      oracle.batched_add_i8(batch, sl, -6, 4, 1, lt, st))
