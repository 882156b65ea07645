"""The gather-pool entry point that takes no workspace and allocates nothing.

Some callers of this library cannot call cudaMalloc: a request thread whose device memory was
all budgeted when the network was loaded, or a plug-in that is only handed buffers.  For them
the library keeps the bag boundaries in a fixed device array of its own.  This test drives that
entry point through the C ABI twice in a row -- the second call with fewer, different bags, so
anything the first call left in the shared array would show -- and requires the results to be
identical to the workspace-taking entry point's (same kernels, so bit for bit).

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.  It passes on its own in a fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from glow_b200 import _lib, ops, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(rows, dim, bags, seed, kind=ops.UINT8_FUSED):
    if kind >= 2:
        table = workloads.fused_table_u4(rows, dim, seed, 0)
    else:
        table = workloads.fused_table_u8(rows, dim, seed, 0)
    wd = np.float16 if kind & 1 else np.float32
    lengths, idx, w = workloads.bags_poisson(bags, 18, 0, 60, rows, seed, 1, np.int64, wd)
    to = lambda a: torch.from_numpy(a).to(DEV)
    return to(table), to(w), to(idx), to(lengths)


def _call_static(table, w, idx, lengths, kind, out, status):
    """Straight through the C ABI, pointer by pointer."""
    rows, in_line = table.shape
    rc = _lib.lib().glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_static_scratch(
        C.c_void_p(out.data_ptr()), C.c_void_p(table.data_ptr()), kind, rows, C.c_void_p(w.data_ptr()),
        C.c_void_p(idx.data_ptr()), 1, C.c_void_p(lengths.data_ptr()), lengths.shape[0], idx.shape[0], in_line,
        ops.out_columns(in_line, kind), int(out.dtype == torch.float16), 0, C.c_void_p(status.data_ptr()),
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc


@pytest.mark.parametrize("kind,dim", [(ops.UINT8_FUSED, 64), (ops.UINT4_FUSED_FP16, 128)])
def test_static_scratch_matches_workspace_entry_point_twice(kind, dim):
    status = ops.new_status(DEV)
    for bags, seed in ((3000, 41), (700, 42)):  # two calls in a row, the second smaller
        table, w, idx, lengths = _inputs(40_000, dim, bags, seed, kind)
        want = ops.fused_rowwise_quantized_sparse_lengths_weighted_sum(table, w, idx, lengths, kind)
        out = torch.full_like(want, float("nan"))
        rc = _call_static(table, w, idx, lengths, kind, out, status)
        torch.cuda.synchronize()
        assert rc == 0, _lib.lib().glowb200_last_error()
        assert int(status.item()) == 0
        assert torch.equal(out, want)


def test_static_scratch_refuses_more_bags_than_it_holds():
    limit = ops.static_scratch_max_segments()
    assert limit == 65536
    table, w, idx, _ = _inputs(1000, 64, 10, 7)
    lengths = torch.zeros(limit + 1, dtype=torch.int32, device=DEV)
    out = torch.empty((limit + 1, 64), device=DEV)
    status = ops.new_status(DEV)
    rc = _call_static(table, w, idx, lengths, ops.UINT8_FUSED, out, status)
    assert rc == 2  # GLOWB200_ERR_UNSUPPORTED
    msg = _lib.lib().glowb200_last_error().decode()
    assert "65537" in msg and "65536" in msg
    # exactly the limit is accepted
    rc = _call_static(table, w, idx, lengths[:limit].contiguous(), ops.UINT8_FUSED, out, status)
    torch.cuda.synchronize()
    assert rc == 0 and not out[:limit].any()
