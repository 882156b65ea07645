"""The C-ABI library loads without a GPU and exports every symbol include/glow_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "glow_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(glowb200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def built():
    from glow_b200 import build
    return build.build()


def test_library_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(built)
    names = _declared()
    assert len(names) >= 6
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_table_matches_header(built):
    from glow_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()
    assert _lib.lib().glowb200_version().startswith(b"glow_b200")


def test_host_side_argument_errors_need_no_gpu(built):
    from glow_b200 import _lib
    l = _lib.lib()
    assert l.glowb200_slws_workspace_bytes(1024, 1) >= 1025 * 8
    assert l.glowb200_slws_workspace_bytes(1024, 4) == 4 * l.glowb200_slws_workspace_bytes(1024, 1)
    # in_line that does not match the column count of the kind
    rc = l.glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum(
        None, None, 0, 10, None, None, 1, None, 0, 0, 70, 64, 0, 0, None, 0, None, None)
    assert rc == 1 and b"in_line_size" in l.glowb200_last_error()
    rc = l.glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum(
        None, None, 7, 10, None, None, 1, None, 0, 0, 72, 64, 0, 0, None, 0, None, None)
    assert rc == 1
    # zero segments is a no-op that needs no device
    rc = l.glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum(
        None, None, 0, 10, None, None, 1, None, 0, 0, 72, 64, 0, 0, None, 0, None, None)
    assert rc == 0
    # Quantize + Transpose: the shuffle is checked on the host; an empty tensor is a no-op
    import ctypes as C
    dims, bad, good = (C.c_int64 * 4)(2, 3, 0, 5), (C.c_int32 * 4)(0, 2, 2, 1), (C.c_int32 * 4)(0, 2, 3, 1)
    rc = l.glowb200_quantize_transpose_i8(None, None, dims, bad, 4, C.c_float(0.1), 0, None)
    assert rc == 1 and b"permutation" in l.glowb200_last_error()
    assert l.glowb200_quantize_transpose_i8(None, None, dims, good, 4, C.c_float(0.1), 0, None) == 0
    assert l.glowb200_transpose(None, None, dims, good, 5, 1, None) == 1
    # the programmatic-launch switch is host state: set, read back, restore
    before = l.glowb200_set_programmatic_launch(0)
    assert l.glowb200_set_programmatic_launch(1) == 0
    assert l.glowb200_set_programmatic_launch(-1) == 1
    assert l.glowb200_set_programmatic_launch(before) in (0, 1)
    l.glowb200_set_programmatic_launch(-1)
