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
