"""The product's host-side parameter derivation (C++ in glow_b200/csrc/quant_params.cu) against
the oracle and the reference's known-answer rules.  Needs no GPU."""
import json
import os

import numpy as np
import pytest

G = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_unit_vectors.json")))


@pytest.fixture(scope="module")
def ops():
    from glow_b200 import build
    build.build()
    from glow_b200 import ops
    return ops


def test_known_answer_scales(ops, oracle):
    g = G["quant_scale_offset"]
    for s in g["scales"] + g["power2_scales"]:
        assert ops.quantize_scale_offset_32to8(np.float32(s)) == oracle.quantize_scale_offset_32to8(np.float32(s))
    for s in g["power2_scales"]:
        pre, post, sc = ops.quantize_scale_offset_32to8(s)
        e = int(np.log2(s))
        assert pre == 0 and ((post, sc) == (0, int(s)) if e > 0 else (post, sc) == (-e, 1))


def test_random_scales_match_oracle(ops, oracle):
    rng = np.random.default_rng(0)
    scales = np.exp(rng.uniform(np.log(1e-9), np.log(1e4), 20000)).astype(np.float32)
    for s in scales[:4000]:
        assert ops.quantize_scale_offset_32to8(s) == oracle.quantize_scale_offset_32to8(s)
    ws = rng.uniform(0.0001, 0.05, 5000).astype(np.float32)
    for bias_scales in (np.float32(5e-4), (np.float32(0.05) * ws).astype(np.float32)):
        got = ops.rowwise_requant_params(ws, 0.05, bias_scales, 0.5)
        want = oracle.rowwise_requant_params(ws, 0.05, bias_scales, 0.5)
        for a, b in zip(got, want):
            np.testing.assert_array_equal(a, b)


def test_choose_quantization_params_known_answers(ops, oracle):
    """tests/unittests/QuantizationTest.cpp:1751-1857."""
    asym = lambda a, b: ops.choose_quantization_params(a, b, ops.ASYMMETRIC)
    sym = lambda a, b: ops.choose_quantization_params(a, b, ops.SYMMETRIC)
    s, o = asym(0.0, 6.0); assert o == -128 and abs(s - 6.0 / 255) < 1e-3
    s, o = asym(-3.0, 3.0); assert o == 0 and abs(s - 6.0 / 255) < 1e-3
    s, o = asym(-2.0, 5.0); assert o == int(2.0 * 255 / 7.0 - 128) and abs(s - 7.0 / 255) < 1e-3
    s, o = asym(2.0, 5.0); assert o == -128 and abs(s - 5.0 / 255) < 1e-3
    s, o = asym(-8.0, -2.0); assert o == 127 and abs(s - 8.0 / 255) < 1e-3
    for rng, want in [((0.0, 6.0), 12.0), ((-3.0, 3.0), 6.0), ((-2.0, 5.0), 10.0), ((2.0, 5.0), 10.0), ((-8.0, -2.0), 16.0)]:
        s, o = sym(*rng)
        assert o == 0 and abs(s - want / 255) < 1e-3
    rng = np.random.default_rng(3)
    for _ in range(2000):
        a, b = np.sort(rng.standard_normal(2).astype(np.float32) * np.float32(10.0) ** rng.integers(-3, 3))
        for schema in range(4):
            got = ops.choose_quantization_params(a, b, schema)
            want = oracle.choose_quantization_params(a, b, schema)
            assert np.float32(got[0]) == want[0] and got[1] == want[1]


def test_tensor_rowwise_quantize_matches_oracle(ops, oracle):
    rng = np.random.default_rng(8)
    w = (rng.standard_normal((200, 333)) * rng.uniform(0.01, 2, (200, 1))).astype(np.float32)
    w[3] = 0
    w[4] = np.abs(w[4])
    for schema in (0, 1, 2):
        got, want = ops.tensor_rowwise_quantize_i8(w, schema), oracle.tensor_rowwise_quantize_i8(w, schema)
        for a, b in zip(got, want):
            np.testing.assert_array_equal(a, b)
    q, sc, off = ops.tensor_rowwise_quantize_i8(w, 0)
    deq = sc[:, None] * (q.astype(np.float32) - off[:, None])
    assert np.max(np.abs(deq - w) / np.maximum(np.abs(w).max(1, keepdims=True), 1e-6)) < 0.01


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
def test_fused_rowwise_quantize_host_matches_oracle(ops, oracle, kind):
    rng = np.random.default_rng(50 + kind)
    for cols in (2, 10, 64, 130):
        table = rng.normal(0, 2, (300, cols)).astype(np.float32)
        table[3] = -1.5            # constant row -> scale 1
        table[4, 1] = 3e4          # wide range
        table[7] *= 1e-12          # range below the equality threshold
        got = ops.fused_rowwise_quantize_host(table, kind)
        np.testing.assert_array_equal(got, oracle.fused_rowwise_quantize(table, kind))


def test_fused_rowwise_quantize_host_known_answer(ops):
    """The fused 4-bit case of the reference's quantisation unit test: a row 0..15 maps to itself."""
    row = np.arange(16, dtype=np.float32)[None, :]
    got = ops.fused_rowwise_quantize_host(row, 3)
    assert got.shape == (1, 12)
    assert got[0, :8].tolist() == [(2 * i) | ((2 * i + 1) << 4) for i in range(8)]
    assert got[0, 8:].view(np.float16).tolist() == [1.0, 0.0]
    with pytest.raises(Exception):
        ops.fused_rowwise_quantize_host(np.zeros((2, 3), np.float32), 2)   # odd column count, 4-bit
