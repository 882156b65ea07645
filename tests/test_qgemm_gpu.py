"""Int8 dense layers on the tensor cores against the CPU oracle: bit-exact.

The oracle itself is checked bit for bit against the reference's own libjit sources
(tests/test_oracle_vs_ref.py); where that build is present it is used here directly as well.
"""
import numpy as np
import pytest
import torch

from glow_b200 import ops, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def make_rwq_fc(rng, M, K, N, w_off_zero=True, in_offset=3, out_offset=0, out_scale=0.5):
    c = dict(
        inp=rng.integers(-128, 128, (M, K)).astype(np.int8),
        w=rng.integers(-127, 128, (N, K)).astype(np.int8),
        bias=rng.integers(-2 ** 16, 2 ** 16, N).astype(np.int32),
        w_off=np.zeros(N, np.int32) if w_off_zero else rng.integers(-20, 20, N).astype(np.int32),
        w_scales=rng.uniform(0.001, 0.02, N).astype(np.float32),
        in_offset=in_offset, out_offset=out_offset, bias_offset=0)
    # keep the outputs inside int8 for every K so the comparison sees real values, not clipping
    eff_out_scale = np.float32(out_scale * np.sqrt(K / 4096.0))
    c["params"] = ops.rowwise_requant_params(c["w_scales"], 0.05, np.float32(5e-4), eff_out_scale)
    return c


def run_rwq(c, flags=0, row_sums=False):
    st = ops.new_status(DEV)
    p = [t(a) for a in c["params"]]
    w = t(c["w"])
    rs = ops.i8_row_sums(w) if row_sums else None
    out = ops.rowwise_quantized_fc(t(c["inp"]), w, t(c["bias"]), t(c["w_off"]), p[:3], p[3:], c["out_offset"],
                                   c["in_offset"], c["bias_offset"], weights_row_sums=rs, flags=flags, status=st)
    torch.cuda.synchronize()
    return out.cpu().numpy(), int(st.item())


def oracle_rwq(oracle, c, threads=8):
    p = c["params"]
    return oracle.rowwise_quantized_fc_i8_i32(c["inp"], c["w"], c["bias"], c["w_off"], p[:3], p[3:], c["out_offset"],
                                              c["in_offset"], c["bias_offset"], threads=threads)


SHAPES = [(128, 128, 256), (128, 512, 256), (256, 4096, 512), (200, 1040, 300), (1, 512, 1), (512, 2208, 1024),
          (33, 16, 7), (384, 256, 64), (130, 272, 40), (1000, 640, 1000)]


@pytest.mark.parametrize("M,K,N", SHAPES)
@pytest.mark.parametrize("w_off_zero", [True, False])
def test_rowwise_fc_bit_exact(oracle, M, K, N, w_off_zero):
    rng = np.random.default_rng(M + 7 * K + 13 * N)
    c = make_rwq_fc(rng, M, K, N, w_off_zero, in_offset=int(rng.integers(-10, 10)), out_offset=int(rng.integers(-5, 5)))
    want = oracle_rwq(oracle, c)
    got, status = run_rwq(c, flags=ops.FC_WEIGHT_OFFSETS_ZERO if w_off_zero else 0)
    assert status == 0
    np.testing.assert_array_equal(got, want)
    assert want.size < 1000 or len(np.unique(want)) > 4
    got2, _ = run_rwq(c, row_sums=True)  # precomputed weight row sums; no hint
    np.testing.assert_array_equal(got2, want)


@pytest.mark.parametrize("M,K,N", [(64, 100, 30), (17, 33, 5), (40, 4095, 9)])
def test_odd_shapes_take_the_any_shape_kernel(oracle, M, K, N):
    rng = np.random.default_rng(K)
    c = make_rwq_fc(rng, M, K, N, w_off_zero=False)
    got, status = run_rwq(c)
    np.testing.assert_array_equal(got, oracle_rwq(oracle, c))


def test_tensor_core_kernel_equals_plain_kernel():
    """Device-side cross-check at a size the CPU oracle would need minutes for."""
    rng = np.random.default_rng(99)
    c = make_rwq_fc(rng, 1024, 4096, 2048, w_off_zero=False)
    a, _ = run_rwq(c)
    b, _ = run_rwq(c, flags=ops.FC_FORCE_ANY_SHAPE_KERNEL)
    np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("pair", ["1", "2"])
@pytest.mark.parametrize("w_off_zero", [True, False])
def test_cta_pair_kernel_equals_plain_kernel(monkeypatch, w_off_zero, pair):
    """The kernel that walks 256-row tiles with pairs of CTAs (one MMA over two SMs), switched on
    through the environment: a ragged last row block (the odd CTA of the last pair has 80 rows)
    and a partial last column tile, against the plain kernel on every element."""
    rng = np.random.default_rng(7)
    c = make_rwq_fc(rng, 2000, 2048, 4000, w_off_zero=w_off_zero)
    flags = ops.FC_WEIGHT_OFFSETS_ZERO if w_off_zero else 0
    single, st0 = run_rwq(c, flags=flags)
    monkeypatch.setenv("GLOWB200_GEMM_PAIR", pair)
    paired, st1 = run_rwq(c, flags=flags)
    monkeypatch.delenv("GLOWB200_GEMM_PAIR")
    plain, _ = run_rwq(c, flags=flags | ops.FC_FORCE_ANY_SHAPE_KERNEL)
    assert st0 == 0 and st1 == 0
    np.testing.assert_array_equal(paired, plain)
    np.testing.assert_array_equal(single, plain)


def test_config2_sampled_rows(oracle):
    """The benchmark's second configuration at full size (M2048 K4096 N4096); the oracle checks
    a seeded sample of 96 batch rows (every output of those rows), the plain kernel all rows."""
    c = workloads.config2()
    params = ops.rowwise_requant_params(c["w_scales"], c["in_scale"], c["bias_scale"], c["out_scale"])
    st = ops.new_status(DEV)
    p = [t(a) for a in params]
    w, inp = t(c["w"]), t(c["inp"])
    args = (inp, w, t(c["bias"]), t(c["w_offsets"]), p[:3], p[3:], c["out_offset"], c["in_offset"], c["bias_offset"])
    out = ops.rowwise_quantized_fc(*args, flags=ops.FC_WEIGHT_OFFSETS_ZERO, status=st)
    plain = ops.rowwise_quantized_fc(*args, flags=ops.FC_FORCE_ANY_SHAPE_KERNEL)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(out, plain)
    rows = np.sort(np.random.default_rng(1).choice(2048, 96, replace=False))
    want = oracle.rowwise_quantized_fc_i8_i32(c["inp"][rows], c["w"], c["bias"], c["w_offsets"], params[:3], params[3:],
                                              c["out_offset"], c["in_offset"], c["bias_offset"], threads=8)
    np.testing.assert_array_equal(out.cpu().numpy()[rows], want)
    # With the configuration's scales (0.05 * U(0.001,0.02) / 0.5) about 60 % of the outputs clip
    # at -128 / 127; the rest cover every int8 value, so the comparison is not vacuous.
    hist = np.bincount(want.astype(np.int32).ravel() + 128, minlength=256)
    assert (hist > 0).sum() == 256 and hist[1:255].sum() > 0.3 * want.size


@pytest.mark.parametrize("M,K,N", [(128, 256, 256), (77, 144, 50), (64, 99, 31), (512, 1024, 1)])
def test_fc_and_matmul_bit_exact(oracle, M, K, N):
    rng = np.random.default_rng(M * N)
    inp = rng.integers(-128, 128, (M, K)).astype(np.int8)
    w = rng.integers(-128, 128, (K, N)).astype(np.int8)
    bias = rng.integers(-5000, 5000, N).astype(np.int32)
    mm = np.float32(0.05) * np.float32(0.01)
    bt = ops.quantize_scale_offset_32to8(np.float32(0.002) / mm)
    ot = ops.quantize_scale_offset_32to8(mm / np.float32(0.3 * np.sqrt(K / 256.0)))
    for w_off in (0, 2):
        want = oracle.fc_i8_i32(inp, w, bias, -4, 3, w_off, 1, bt, ot, threads=4)
        got = ops.fully_connected_i8(t(inp), t(w), t(bias), -4, 3, w_off, 1, bt, ot)
        np.testing.assert_array_equal(got.cpu().numpy(), want)
        wt = t(np.ascontiguousarray(w.T))
        got = ops.fully_connected_i8(t(inp), None, t(bias), -4, 3, w_off, 1, bt, ot, weights_transposed=wt)
        np.testing.assert_array_equal(got.cpu().numpy(), want)
        want = oracle.matmul_i8(inp, w, 5, -3, w_off, ot, threads=4)
        got = ops.matmul_i8(t(inp), t(w), 5, -3, w_off, ot)
        np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_row_sums():
    rng = np.random.default_rng(2)
    for rows, K in [(300, 4096), (17, 100), (1, 16)]:
        x = rng.integers(-128, 128, (rows, K)).astype(np.int8)
        np.testing.assert_array_equal(ops.i8_row_sums(t(x)).cpu().numpy(), x.astype(np.int32).sum(1))


@pytest.mark.parametrize("M,K,N", [(256, 512, 256), (64, 100, 30)])
def test_int8_bias_forms(oracle, M, K, N):
    """The reference's _i8_i8 entry points: an int8 bias goes through the same arithmetic as an
    int32 bias holding the same values (tensor-core and any-shape kernels)."""
    rng = np.random.default_rng(M + N)
    c = make_rwq_fc(rng, M, K, N, True)
    c["bias"] = rng.integers(-128, 128, N).astype(np.int32)
    c["bias_offset"] = 5
    # a bias scale that makes the small int8 bias matter in the result
    c["params"] = ops.rowwise_requant_params(c["w_scales"], 0.05, np.float32(0.8), np.float32(0.5 * np.sqrt(K / 4096.0)))
    want = oracle_rwq(oracle, c)
    st = ops.new_status(DEV)
    p = [t(a) for a in c["params"]]
    got = ops.rowwise_quantized_fc(t(c["inp"]), t(c["w"]), t(c["bias"].astype(np.int8)), t(c["w_off"]), p[:3], p[3:],
                                   c["out_offset"], c["in_offset"], c["bias_offset"], status=st).cpu().numpy()
    np.testing.assert_array_equal(got, want)
    got32, _ = run_rwq(c)
    np.testing.assert_array_equal(got32, want)
    assert int(st.item()) == 0
    # per-tensor FullyConnected
    w_kn = np.ascontiguousarray(c["w"].T)
    bt, ot = oracle.quantize_scale_offset_32to8(np.float32(0.7)), oracle.quantize_scale_offset_32to8(np.float32(0.004))
    want = oracle.fc_i8_i32(c["inp"], w_kn, c["bias"], 2, c["in_offset"], 1, c["bias_offset"], bt, ot)
    got = ops.fully_connected_i8(t(c["inp"]), t(w_kn), t(c["bias"].astype(np.int8)), 2, c["in_offset"], 1,
                                 c["bias_offset"], bt, ot).cpu().numpy()
    np.testing.assert_array_equal(got, want)


def test_bounded_wait_gives_up_and_leaves_the_context_usable(oracle):
    """A device-side wait that cannot complete runs out after its limit, reports through the status
    word and returns; the next launch on the same context works."""
    st = ops.new_status(DEV)
    gave_up = ops.wait_limit_selftest(2_000_000, st)      # about a millisecond of SM clocks
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 2
    assert int(st.item()) == ops.STATUS_WAIT_TIMEOUT
    rng = np.random.default_rng(1)
    c = make_rwq_fc(rng, 128, 256, 256)
    got, status = run_rwq(c)
    assert status == 0
    np.testing.assert_array_equal(got, oracle_rwq(oracle, c))
