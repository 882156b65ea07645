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
