"""The CPU oracle against the expected tensors of the reference's own unit tests
(tests/golden/reference_unit_vectors.json, transcribed from OperatorTest.cpp /
QuantizationTest.cpp of pytorch/glow)."""
import json
import os

import numpy as np
import pytest

G = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_unit_vectors.json")))

SLWS_CASES = ["frwq_slws_single_column", "frwq_sls_two_column", "frwq_slws_two_column",
              "frwq_slws_all_lengths_one"]


def _variants(case):
    return [(case, i) for i in range(len(G[case]["variants"]))]


@pytest.mark.parametrize("case,vi", sum((_variants(c) for c in SLWS_CASES), []))
@pytest.mark.parametrize("idx_dtype", [np.int64, np.int32])
def test_slws_golden(oracle, case, vi, idx_dtype):
    g, v = G[case], G[case]["variants"][vi]
    kind = v["kind"]
    table = oracle.fused_rowwise_quantize(np.array(g["data"], np.float32), kind)
    idx = np.array(g["indices"], idx_dtype)
    out = oracle.frwq_slws_interp(table, kind, g["weights"], idx, g["lengths"], fp16_acc=v["fp16_acc"])
    exp = np.array(g["expected"], np.float32)
    assert out.dtype == (np.float16 if kind & 1 else np.float32)
    np.testing.assert_allclose(out.astype(np.float32), exp, atol=v["tol"], rtol=0)
    if kind == 0:
        # CPU-backend (libjit) form of the same operator
        out2 = oracle.frwq_slws_u8_f32(table, g["weights"], idx, g["lengths"])
        np.testing.assert_allclose(out2, exp, atol=v["tol"], rtol=0)


@pytest.mark.parametrize("vi", range(3))
@pytest.mark.parametrize("mode", ["no_end", "with_end", "partial"])
def test_embedding_bag_golden(oracle, vi, mode):
    g = G["embedding_bag_byte_rowwise_offsets"]
    v = g["variants"][vi]
    kind = v["kind"]
    table = oracle.fused_rowwise_quantize(np.array(g["data"], np.float32), kind)
    w = np.array(g["weights"], np.float32)
    idx = np.array(g["indices"], np.int32)
    exp = np.array(g["expected"], np.float32)
    if mode == "no_end":
        off, has_end = np.array(g["offsets_no_end"], np.int32), False
    else:
        off, has_end = np.array(g["offsets_with_end"], np.int32), True
    if mode == "partial":
        p = g["partial"]
        w = np.concatenate([w, np.zeros(p["weights_len"] - w.size, np.float32)])
        idx = np.concatenate([idx, np.zeros(p["indices_len"] - idx.size, np.int32)])
        off = np.concatenate([off, np.zeros(p["offsets_len"] - off.size, np.int32)])
        exp = np.array(p["expected"], np.float32)
    out = oracle.embedding_bag_byte_rowwise_offsets(table, kind, w, idx, off, has_end, fp16_acc=v["fp16_acc"])
    np.testing.assert_allclose(out.astype(np.float32), exp, atol=v["tol"], rtol=0)


def test_quant_scale_offset_known_answers(oracle):
    g = G["quant_scale_offset"]
    for s in g["scales"]:
        s = np.float32(s)
        pre, post, sc = oracle.quantize_scale_offset_32to8(s)
        for inp in range(-128, 127):
            x = int(np.round(np.float64(inp) / np.float64(s)))  # C round(): half away from zero
            x = int(np.sign(inp) * np.floor(abs(np.float64(inp) / np.float64(s)) + 0.5))
            if not (-2 ** 31 <= x < 2 ** 31):
                continue
            got = oracle.scale32(x, pre, post, sc, 0)
            assert abs(got - inp) <= 1, (float(s), inp, x, pre, post, sc, got)


def test_quant_scale_offset_power_of_two(oracle):
    for s in G["quant_scale_offset"]["power2_scales"]:
        pre, post, sc = oracle.quantize_scale_offset_32to8(s)
        e = int(np.log2(s))
        assert pre == 0
        if e > 0:
            assert (post, sc) == (0, int(s))
        else:
            assert (post, sc) == (-e, 1)
        for inp in range(-128, 127):
            x = int(np.sign(inp) * np.floor(abs(inp / s) + 0.5))
            assert abs(oracle.scale32(x, pre, post, sc, 0) - inp) <= 1


def test_fp16_conversion_matches_ieee(oracle):
    rng = np.random.default_rng(5)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 4000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 5.96e-8, 2.98e-8, 2.9802322e-08, 6.1e-5,
                  6.1035156e-05, 1.0009766, 1.0004883, 1.0014648], np.float32)])
    got = oracle.f32_to_f16_bits(vals)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    np.testing.assert_array_equal(got, want)
    back = np.array([oracle.lib().orc_f16_to_f32(int(h)) for h in range(0, 0x7c00, 7)], np.float32)
    np.testing.assert_array_equal(back, np.arange(0, 0x7c00, 7, dtype=np.uint16).view(np.float16).astype(np.float32))


def test_fused_4bit_roundtrip(oracle):
    """Mirror of fused4BitRowwiseQuantizationTest (QuantizationTest.cpp:440-519): values on the
    row's own 16-level grid survive quantize -> dequantize."""
    rng = np.random.default_rng(11)
    for kind in (2, 3):
        rows, cols = 12, 32
        lo = rng.uniform(-2, 0, (rows, 1)).astype(np.float32)
        step = np.float32(0.125)
        q = rng.integers(0, 16, (rows, cols))
        q[:, 0], q[:, 1] = 0, 15
        data = (lo + q * step).astype(np.float32)
        table = oracle.fused_rowwise_quantize(data, kind)
        ones = np.ones(rows, np.float16 if kind & 1 else np.float32)
        out = oracle.frwq_slws_interp(table, kind, ones, np.arange(rows, dtype=np.int64), np.ones(rows, np.int32))
        np.testing.assert_allclose(out.astype(np.float32), data, atol=0.02 if kind & 1 else 1e-5)


from split_embedding_cases import CASES as SPLIT_CASES, case_inputs as split_case_inputs


@pytest.mark.parametrize("name", SPLIT_CASES)
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_int_nbit_split_embedding_bags_golden(oracle, name, idx_dtype):
    """OperatorTest.cpp:21308-21762: table-batched embedding bags, all sixteen cases."""
    a, expected, tol = split_case_inputs(name, idx_dtype)
    out = oracle.int_nbit_split_embedding_bags(**a)
    assert out.dtype == (np.float16 if a["out_fp16"] else np.float32)
    np.testing.assert_allclose(out.astype(np.float32), expected, atol=tol, rtol=0)


def _dyn_fc_case(c):
    x = np.array(c["input"], np.float16)
    w = np.array(c["weights"], np.int8)
    n = w.shape[1]
    scales = np.array(c["scales"], np.float32) if "scales" in c else np.full(n, c["weights_scale"], np.float32)
    offsets = np.array(c["offsets"], np.int32) if "offsets" in c else np.full(n, c["weights_offset"], np.int32)
    return x, w, np.array(c["bias"], np.float32), scales, offsets


@pytest.mark.parametrize("ci", range(3))
def test_dynamic_quantized_fc_golden(oracle, ci):
    """OperatorTest.cpp:7787-7886: the three dynamically quantized FC cases."""
    c = G["dynamic_quantized_fc"]["cases"][ci]
    out = oracle.dynamic_rowwise_quantized_fc(*_dyn_fc_case(c))
    np.testing.assert_allclose(out.astype(np.float32), np.array(c["expected"], np.float32), atol=c["tol"], rtol=0)
