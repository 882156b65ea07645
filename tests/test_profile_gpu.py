"""The quantization-profile kernels against the oracle (itself checked against the reference's
libjit_quantization_profile): running min / max and histogram, bit for bit, over sequences of
tensors whose range grows, shrinks and collapses."""
import numpy as np
import pytest
import torch

from glow_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("bins", [0, 1, 10, 2000, 10000])
def test_profile_sequence(oracle, bins):
    rng = np.random.default_rng(3 + bins)
    ci_o = np.array([np.finfo(np.float32).max, np.finfo(np.float32).min], np.float32)
    h_o = np.zeros(bins, np.float32)
    ci_d = torch.from_numpy(ci_o.copy()).to(DEV)
    h_d = torch.zeros(max(bins, 0), dtype=torch.float32, device=DEV)
    for scale, shift, n in [(1.0, 0.0, 50000), (0.3, 0.1, 777), (4.0, -2.0, 300000), (4.0, 5.0, 3000), (0.0, 1.5, 100),
                            (20.0, 0.0, 1), (1.0, 0.0, 1 << 20)]:
        x = (rng.normal(0, 1, n) * scale + shift).astype(np.float32)
        ci_o, h_o = oracle.quantization_profile(x, ci_o, h_o)
        ops.quantization_profile(torch.from_numpy(x).to(DEV), ci_d, h_d)
        np.testing.assert_array_equal(ci_d.cpu().numpy().view(np.uint32), ci_o.view(np.uint32))
        np.testing.assert_array_equal(h_d.cpu().numpy().view(np.uint32), h_o.view(np.uint32))


def test_counter_saturates_like_a_float():
    """A float counter stops at 2^24; the kernel adds whole counts and must stop there too."""
    ci = torch.tensor([0.0, 1.0], device=DEV)
    hist = torch.tensor([16777210.0, 5.0], device=DEV)
    x = torch.cat([torch.zeros(100, device=DEV), torch.ones(3, device=DEV)])
    ops.quantization_profile(x, ci, hist)
    assert hist.tolist() == [16777216.0, 8.0]


@pytest.mark.parametrize("schema", [ops.ASYMMETRIC, ops.SYMMETRIC, ops.SYMMETRIC_WITH_UNSIGNED, ops.SYMMETRIC_WITH_POWER2_SCALE])
@pytest.mark.parametrize("rows,cols", [(1, 1), (37, 100), (512, 2208), (64, 4097)])
def test_rowwise_weight_quantiser_on_device(oracle, schema, rows, cols):
    """tensorRowwiseQuantization on the device gives the bytes and parameters of the oracle (and
    of the host function the library also exports)."""
    rng = np.random.default_rng(rows + cols + schema)
    w = (rng.normal(0, 1, (rows, cols)) * rng.uniform(0.01, 3, (rows, 1))).astype(np.float32)
    if rows > 3:
        w[1] = 0
        w[2] = np.abs(w[2])
        w[3, :] = 0.25           # a constant row: scale a power of two candidate
    q, sc, off = ops.tensor_rowwise_quantize_i8_device(torch.from_numpy(w).to(DEV), schema)
    want_q, want_sc, want_off = oracle.tensor_rowwise_quantize_i8(w, schema)
    np.testing.assert_array_equal(sc.cpu().numpy().view(np.uint32), want_sc.view(np.uint32))
    np.testing.assert_array_equal(off.cpu().numpy(), want_off)
    np.testing.assert_array_equal(q.cpu().numpy(), want_q)
    hq, hsc, hoff = ops.tensor_rowwise_quantize_i8(w, schema)
    np.testing.assert_array_equal(hq, want_q)
    # the same elements again, parameters given
    q2 = ops.quantize_rows_i8_device(torch.from_numpy(w).to(DEV), sc, off)
    np.testing.assert_array_equal(q2.cpu().numpy(), want_q)
