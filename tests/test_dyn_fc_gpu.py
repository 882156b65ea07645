"""Parity of the dynamically quantized fully connected layers through the C ABI: every input row
quantized on the device with its own symmetric parameters, int32 sums from the tensor cores (or
the any-shape kernel), floating-point rescale -- bit for bit against the oracle's restatement of
the Interpreter (InterpreterNodes.cpp:4677-4790)."""
import numpy as np
import pytest
import torch

from glow_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def make(seed, M, K, N, zero_offsets):
    rng = np.random.default_rng(seed)
    x = (rng.normal(0, 1, (M, K)) * rng.uniform(0.01, 30, (M, 1))).astype(np.float16)
    x[M // 2] = 0                      # a row of zeros: the scale falls back to 0.1
    if M > 2:
        x[1] = np.abs(x[1])            # one-sided rows
        x[2] = -np.abs(x[2])
    w = rng.integers(-128, 128, (K, N), dtype=np.int8)
    bias = rng.normal(0, 2, N).astype(np.float32)
    scales = rng.uniform(0.001, 0.02, N).astype(np.float32)
    offsets = np.zeros(N, np.int32) if zero_offsets else rng.integers(-20, 20, N).astype(np.int32)
    return x, w, bias, scales, offsets


@pytest.mark.parametrize("M,K,N", [(5, 64, 48), (130, 256, 300), (64, 100, 33), (257, 1024, 512), (1, 16, 1),
                                   (128, 2048, 64), (33, 4096, 40), (16, 8192, 32), (9, 4104, 16), (7, 9000, 8)])
@pytest.mark.parametrize("zero_offsets", [True, False])
@pytest.mark.parametrize("transposed", [False, True])
def test_dynamic_rowwise_quantized_fc(oracle, M, K, N, zero_offsets, transposed):
    x, w, bias, scales, offsets = make(M + K + N, M, K, N, zero_offsets)
    want = oracle.dynamic_rowwise_quantized_fc(x, w, bias, scales, offsets)
    st = ops.new_status(DEV)
    kw = {}
    if transposed:
        kw["weights_transposed"] = t(w.T.copy())
    got = ops.dynamic_rowwise_quantized_fc(t(x), None if transposed else t(w), t(bias), t(scales), t(offsets),
                                           flags=ops.FC_WEIGHT_OFFSETS_ZERO if zero_offsets else 0, status=st, **kw)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))
    assert int(st.item()) == 0
    # the any-shape kernel on the same inputs
    got = ops.dynamic_rowwise_quantized_fc(t(x), t(w), t(bias), t(scales), t(offsets),
                                           flags=ops.FC_FORCE_ANY_SHAPE_KERNEL, status=st)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))
    assert int(st.item()) == 0


@pytest.mark.parametrize("M,K,N", [(33, 128, 70), (9, 50, 20)])
@pytest.mark.parametrize("w_offset", [0, 7])
def test_dynamic_quantized_fc(oracle, M, K, N, w_offset):
    x, w, bias, _, _ = make(3 * M + K, M, K, N, True)
    w_scale = 0.0123
    want = oracle.dynamic_rowwise_quantized_fc(x, w, bias, np.full(N, w_scale, np.float32), np.full(N, w_offset, np.int32))
    st = ops.new_status(DEV)
    got = ops.dynamic_quantized_fc(t(x), t(w), t(bias), w_scale, w_offset, status=st)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))
    assert int(st.item()) == 0


@pytest.mark.parametrize("ci", range(3))
def test_reference_unit_cases(oracle, ci):
    """The reference's own operator tests (OperatorTest.cpp:7787-7886) through the C ABI."""
    import json
    import os
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_unit_vectors.json")))
    c = g["dynamic_quantized_fc"]["cases"][ci]
    x, w = np.array(c["input"], np.float16), np.array(c["weights"], np.int8)
    bias = np.array(c["bias"], np.float32)
    if "scales" in c:
        got = ops.dynamic_rowwise_quantized_fc(t(x), t(w), t(bias), t(np.array(c["scales"], np.float32)),
                                               t(np.array(c["offsets"], np.int32)))
    else:
        got = ops.dynamic_quantized_fc(t(x), t(w), t(bias), c["weights_scale"], c["weights_offset"])
    np.testing.assert_allclose(got.cpu().numpy().astype(np.float32), np.array(c["expected"], np.float32),
                               atol=c["tol"], rtol=0)
