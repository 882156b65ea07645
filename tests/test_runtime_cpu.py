"""Host runtime without a GPU: building and compiling functions, and the errors that do not need
a device."""
import numpy as np
import pytest

from glow_b200 import runtime
from glow_b200._lib import GlowB200Error


@pytest.fixture(scope="module", autouse=True)
def built():
    from glow_b200 import build
    build.build()


def test_compile_lays_out_slabs_and_derives_constants():
    f = runtime.Function("fc")
    N, K, M = 8, 32, 4
    w = f.constant("w", np.ones((N, K), np.int8))
    sc = f.constant("scales", np.full(N, 0.01, np.float32))
    off = f.constant("offsets", np.zeros(N, np.int32))
    b = f.constant("bias", np.zeros(N, np.int32))
    x = f.placeholder("x", M * K)
    y = f.placeholder("y", M * N)
    f.rowwise_fc(y, x, w, sc, off, b, M=M, K=K, N=N, in_tqp=(0.05, 3), bias_tqp=(5e-4, 0), out_tqp=(0.5, 0))
    before = N * K + 3 * N * 4
    f.compile()
    # six per-row triples and the weight row sums were added as constants, each slot 64-byte aligned
    assert f.constant_bytes >= before + 7 * N * 4
    assert f.constant_bytes % 64 == 0
    with pytest.raises(GlowB200Error):
        f.compile()  # already compiled


def test_building_errors():
    f = runtime.Function("bad")
    f.placeholder("x", 16)
    with pytest.raises(GlowB200Error, match="already exists"):
        f.placeholder("x", 16)
    f.instruction(99, [0], [1], [])
    with pytest.raises(GlowB200Error, match="unsupported kind"):
        f.compile()
    g = runtime.Function("bad2")
    a = g.placeholder("a", 8)
    g.instruction(runtime.MAXSPLAT, [a, a], [8])  # one attribute short
    with pytest.raises(GlowB200Error, match="malformed"):
        g.compile()
    h = runtime.Function("bad3")
    with pytest.raises(GlowB200Error, match="no such symbol"):
        h.instruction(runtime.COPY, [5, 6], [4])


def test_device_manager_needs_init():
    dm = runtime.DeviceManager(0, 1 << 20)
    f = runtime.Function("f")
    a = f.placeholder("a", 8)
    f.copy(a, a, nbytes=8)
    f.compile()
    with pytest.raises(GlowB200Error, match="not initialised"):
        dm.add_network(f)
    assert dm.maximum_memory == 1 << 20 and dm.available_memory == 1 << 20
    assert dm.is_memory_available(1 << 20) and not dm.is_memory_available((1 << 20) + 1)


def test_new_instruction_kinds_compile_and_reject_malformed_forms():
    """Arithmetic glue, table-batched bags and the dynamically quantized FC: compile derives the
    integer triples (three or six more attributes) and sizes the workspace; wrong operand or
    attribute counts are refused."""
    from glow_b200 import ops
    f = runtime.Function("arith")
    a, b, c = f.placeholder("a", 64), f.placeholder("b", 64), f.placeholder("c", 64)
    f.binary(ops.BINARY_MIN, c, a, b, n=64, lhs_tqp=(0.02, 1), rhs_tqp=(0.03, -2), dest_tqp=(0.05, 0))
    f.muldiv(True, c, a, b, n=64, lhs_tqp=(0.02, 1), rhs_tqp=(0.03, -2), dest_tqp=(0.05, 0))
    f.batched_add(c, a, b, num_slices=4, slice_size=16, batch_tqp=(0.02, 1), slice_tqp=(0.03, -2), dest_tqp=(0.05, 0))
    x = f.placeholder("x", 8 * 32 * 2)
    w = f.constant("w", np.ones((32, 16), np.int8))
    bias = f.constant("bias", np.zeros(16, np.float32))
    y = f.placeholder("y", 8 * 16 * 2)
    f.dynamic_quantized_fc(y, x, w, bias, M=8, K=32, N=16, weights_tqp=(0.01, 0))
    f.compile()
    g = runtime.Function("bad_dyn")
    x = g.placeholder("x", 64)
    sc = g.constant("scales", np.ones(4, np.float32))
    g.instruction(runtime.DYN_QUANTIZED_FC, [x, x, x, x, sc, -1], [2, 16, 4, 0], [0.0])   # scales without offsets
    with pytest.raises(GlowB200Error, match="both scales and offsets"):
        g.compile()
    h = runtime.Function("bad_split")
    x = h.placeholder("x", 64)
    h.instruction(runtime.SPLIT_EMBEDDING, [x] * 9, [0] * 13)                               # an operand short
    with pytest.raises(GlowB200Error, match="malformed SPLIT_EMBEDDING"):
        h.compile()
    k = runtime.Function("bad_binary")
    x = k.placeholder("x", 64)
    k.instruction(runtime.BINARY_I8, [x, x, x], [64, 0, 0, 0], [1.0, 1.0, 1.0])            # the operator is missing
    with pytest.raises(GlowB200Error, match="malformed BINARY_I8"):
        k.compile()


def _fc_function(name, *, y_bytes=None, scales=True, M=4, K=32, N=8):
    f = runtime.Function(name)
    w = f.constant("w", np.ones((N, K), np.int8))
    sc = f.constant("scales", np.full(N, 0.01, np.float32)) if scales else -1
    off = f.constant("offsets", np.zeros(N, np.int32))
    b = f.constant("bias", np.zeros(N, np.int32))
    x = f.placeholder("x", M * K)
    y = f.placeholder("y", M * N if y_bytes is None else y_bytes)
    return f, (y, x, w, sc, off, b), dict(M=M, K=K, N=N, in_tqp=(0.05, 3), bias_tqp=(5e-4, 0), out_tqp=(0.5, 0))


def test_compile_rejects_what_would_leave_a_symbol():
    """An instruction is checked against the byte sizes of the symbols it names: nothing that
    would read or write outside one of them compiles."""
    f, ops_, kw = _fc_function("short_dest", y_bytes=4 * 8 - 1)
    f.rowwise_fc(*ops_, **kw)
    with pytest.raises(GlowB200Error, match="smaller than"):
        f.compile()
    # a required operand left out
    f, ops_, kw = _fc_function("no_scales", scales=False)
    f.rowwise_fc(*ops_, **kw)
    with pytest.raises(GlowB200Error, match="is required"):
        f.compile()
    # a constant as destination
    f, ops_, kw = _fc_function("const_dest")
    f.rowwise_fc(ops_[2], *ops_[1:], **dict(kw, M=8, K=32, N=8))
    with pytest.raises(GlowB200Error, match="smaller than|is a constant"):
        f.compile()
    g = runtime.Function("copy_into_const")
    c = g.constant("c", np.zeros(16, np.int8))
    a = g.placeholder("a", 16)
    g.copy(c, a, nbytes=16)
    with pytest.raises(GlowB200Error, match="is a constant"):
        g.compile()
    # copies, element-wise kernels and insert-tensor are bounded too
    g = runtime.Function("long_copy")
    a, b = g.placeholder("a", 16), g.placeholder("b", 8)
    g.copy(a, b, nbytes=16)
    with pytest.raises(GlowB200Error, match="smaller than"):
        g.compile()
    g = runtime.Function("insert")
    a, b = g.placeholder("a", 64), g.placeholder("b", 32)
    g.insert_tensor(a, b, rows=4, width_bytes=8, dest_pitch_bytes=16, dest_offset_bytes=12)  # last row ends at 68
    with pytest.raises(GlowB200Error, match="smaller than"):
        g.compile()
    g = runtime.Function("insert_ok")
    a, b = g.placeholder("a", 64), g.placeholder("b", 32)
    g.insert_tensor(a, b, rows=4, width_bytes=8, dest_pitch_bytes=16, dest_offset_bytes=8)
    g.compile()


def test_convolution_group_is_checked_before_it_divides():
    f = runtime.Function("conv_group0")
    ids = [f.placeholder("y", 16), f.placeholder("x", 16), f.constant("w", np.zeros(16, np.int8)),
           f.constant("b", np.zeros(4, np.int32)), f.constant("fs", np.ones(4, np.float32)),
           f.constant("fo", np.zeros(4, np.int32)), f.constant("bs", np.ones(4, np.float32)),
           f.constant("bo", np.zeros(4, np.int32))]
    ia = [1, 2, 2, 4, 2, 2, 4, 1, 1, 1, 1, 0, 0, 0, 0, 0, 1, 1, 0, 0, 0]  # group = 0
    f.instruction(runtime.CWQ_CONV, ids, ia, [0.1, 0.1])
    with pytest.raises(GlowB200Error, match="group"):
        f.compile()


def test_views_are_checked_against_their_symbol():
    g = runtime.Function("view_too_far")
    a, b = g.placeholder("a", 64), g.placeholder("b", 32)
    g.copy((a, 48), b, nbytes=32)  # 48 + 32 > 64
    with pytest.raises(GlowB200Error, match="smaller than"):
        g.compile()
    g = runtime.Function("view_ok")
    a, b = g.placeholder("a", 64), g.placeholder("b", 32)
    g.copy((a, 32), b, nbytes=32)
    g.compile()
    assert g.batched_pooling_launches == 0


def test_quantize_feeding_only_a_transpose_becomes_one_kernel():
    """Quantize into an activation that nothing but the Transpose right behind it reads is absorbed by
    that Transpose at compile; a second reader of the activation keeps the two kernels."""
    def build(extra_reader):
        f = runtime.Function("stem" + str(int(extra_reader)))
        n = 2 * 3 * 4 * 5
        x = f.placeholder("x", n * 4)
        q = f.activation("q", n)
        y = f.placeholder("y", n)
        f.quantize(q, x, n=n, tqp=(0.05, 3))
        f.transpose(y, q, dims=(2, 3, 4, 5), shuffle=(0, 2, 3, 1), elem_bytes=1)
        if extra_reader:
            z = f.placeholder("z", n)
            f.copy(z, q, nbytes=n)
        return f.compile()
    assert build(False).fused_quantize_transposes == 1
    assert build(True).fused_quantize_transposes == 0
