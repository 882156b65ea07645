"""Operator front end over the C ABI, for callers that hold torch CUDA tensors.

Names and argument meaning follow the reference's kernel entry points
(lib/LLVMIRCodeGen/libjit/libjit.cpp) and node creators (lib/Graph/Graph.cpp); torch is used
only for device memory and streams.  Every function enqueues on torch's current stream.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import SlwsJob, check

UINT8_FUSED, UINT8_FUSED_FP16, UINT4_FUSED, UINT4_FUSED_FP16 = 0, 1, 2, 3

STATUS_INDEX_OUT_OF_RANGE = 1
STATUS_LENGTHS_OVERRUN = 2
STATUS_NEGATIVE_LENGTH = 4
STATUS_BAD_OFFSETS = 8
STATUS_WAIT_TIMEOUT = 16
STATUS_UNSUPPORTED_TABLE = 32


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _cuda(t, name, dtypes=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    if dtypes is not None and t.dtype not in dtypes:
        raise TypeError("%s has dtype %s, expected one of %s" % (name, t.dtype, dtypes))
    return t


def out_columns(in_line_size, kind):
    """Columns of the result for a fused table whose rows are in_line_size bytes."""
    payload = in_line_size - (4 if (kind & 1) else 8)
    return payload * 2 if kind >= 2 else payload


def result_dtype(kind):
    """UInt8FusedQTy/UInt4FusedQTy -> fp32, the FP16 kinds -> fp16 (lib/Graph/Graph.cpp:2446-2476)."""
    return torch.float16 if (kind & 1) else torch.float32


def slws_workspace_bytes(max_segments, num_jobs=1):
    return int(_lib.lib().glowb200_slws_workspace_bytes(int(max_segments), int(num_jobs)))


def new_status(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


def _workspace(workspace, need, device):
    if workspace is None:
        return torch.empty(max(need, 8), dtype=torch.uint8, device=device)
    _cuda(workspace, "workspace")
    return workspace


def fused_rowwise_quantized_sparse_lengths_weighted_sum(data, weights, indices, lengths, kind=UINT8_FUSED, *,
                                                        use_fp16_accumulation=False, out=None, status=None,
                                                        workspace=None, num_indices=None, out_line=None,
                                                        low_latency=False):
    """FusedRowwiseQuantizedSparseLengthsWeightedSum.  data: uint8 [rows, in_line] fused table;
    weights: result dtype [n]; indices: int32/int64 [n]; lengths: int32 [segments].
    out_line: columns of the result when the rows are padded (see pad_fused_rows); default: the
    whole row is payload + scale/offset."""
    _cuda(data, "data", (torch.uint8,))
    _cuda(indices, "indices", (torch.int32, torch.int64))
    _cuda(lengths, "lengths", (torch.int32,))
    rows, in_line = data.shape
    out_line = out_columns(in_line, kind) if out_line is None else int(out_line)
    odt = result_dtype(kind) if out is None else out.dtype
    _cuda(weights, "weights", (odt,))
    segments = lengths.shape[0]
    if out is None:
        out = torch.empty((segments, out_line), dtype=odt, device=data.device)
    n = indices.shape[0] if num_indices is None else int(num_indices)
    need = slws_workspace_bytes(segments, 1)
    ws = _workspace(workspace, need, data.device)
    if low_latency:   # a warp per bag: for small requests; another summation order (see the header)
        if use_fp16_accumulation:
            raise ValueError("the low-latency form accumulates in fp32")
        check(_lib.lib().glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_low_latency(
            _p(out), _p(data), kind, rows, _p(weights), _p(indices), int(indices.dtype == torch.int64), _p(lengths),
            segments, n, in_line, out_line, int(odt == torch.float16), _p(ws), ws.numel(), _p(status), _stream()))
        return out
    check(_lib.lib().glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum(
        _p(out), _p(data), kind, rows, _p(weights), _p(indices), int(indices.dtype == torch.int64), _p(lengths),
        segments, n, in_line, out_line, int(odt == torch.float16), int(use_fp16_accumulation), _p(ws), ws.numel(),
        _p(status), _stream()))
    return out


def fused_rowwise_quantized_sparse_lengths_weighted_sum_static_scratch(data, weights, indices, lengths,
                                                                       kind=UINT8_FUSED, *, out,
                                                                       use_fp16_accumulation=False, status=None,
                                                                       num_indices=None):
    """The same operator for callers that must not allocate: `out` is required, no workspace is
    taken (the bag boundaries go into an array built into the library) and nothing is allocated
    here either.  At most static_scratch_max_segments() bags; calls that may overlap on the GPU
    must be serialised by the caller."""
    rows, in_line = data.shape
    n = indices.shape[0] if num_indices is None else int(num_indices)
    check(_lib.lib().glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_static_scratch(
        _p(out), _p(data), kind, rows, _p(weights), _p(indices), int(indices.dtype == torch.int64), _p(lengths),
        lengths.shape[0], n, in_line, out_columns(in_line, kind), int(out.dtype == torch.float16),
        int(use_fp16_accumulation), _p(status), _stream()))
    return out


def static_scratch_max_segments():
    return int(_lib.lib().glowb200_slws_static_scratch_max_segments())


def fused_rowwise_quantized_sparse_lengths_sum(data, indices, lengths, kind=UINT8_FUSED, **kw):
    """Unweighted form = weighted with weights of one (lib/Optimizer/Lower/Lower.cpp:1590-1606)."""
    odt = result_dtype(kind)
    ones = torch.ones(indices.shape[0], dtype=odt, device=data.device)
    return fused_rowwise_quantized_sparse_lengths_weighted_sum(data, ones, indices, lengths, kind, **kw)


def embedding_bag_byte_rowwise_offsets(data, weights, indices, offsets, kind=UINT8_FUSED, *, has_end_offset=True,
                                       use_fp16_accumulation=False, out=None, status=None, workspace=None,
                                       num_indices=None):
    """EmbeddingBagByteRowwiseOffsets: bags given by offsets (same integer type as indices)."""
    _cuda(data, "data", (torch.uint8,))
    _cuda(indices, "indices", (torch.int32, torch.int64))
    _cuda(offsets, "offsets", (indices.dtype,))
    rows, in_line = data.shape
    out_line = out_columns(in_line, kind)
    odt = result_dtype(kind) if out is None else out.dtype
    _cuda(weights, "weights", (odt,))
    num_offsets = offsets.shape[0]
    segments = num_offsets - 1 if has_end_offset else num_offsets
    if out is None:
        out = torch.empty((max(segments, 0), out_line), dtype=odt, device=data.device)
    n = indices.shape[0] if num_indices is None else int(num_indices)
    need = slws_workspace_bytes(max(segments, 0), 1)
    ws = _workspace(workspace, need, data.device)
    check(_lib.lib().glowb200_embedding_bag_byte_rowwise_offsets(
        _p(out), _p(data), kind, rows, _p(weights), _p(indices), _p(offsets), int(indices.dtype == torch.int64),
        num_offsets, n, in_line, out_line, int(has_end_offset), int(odt == torch.float16),
        int(use_fp16_accumulation), _p(ws), ws.numel(), _p(status), _stream()))
    return out


EST_FLOAT, EST_FLOAT16, EST_INT8, EST_INT4 = 0, 1, 2, 3   # SplitEmbeddingSparseType
EP_SUM, EP_MEAN, EP_NONE = 0, 1, 2                         # SplitEmbeddingPoolingMode
PLACEMENT_DEVICE, PLACEMENT_MANAGED, PLACEMENT_MANAGED_CACHING, PLACEMENT_HOST = 0, 1, 2, 3


def split_embedding_row_bytes(num_dims, weights_ty, *, scale_offset_is_fp32=False, row_alignment=16):
    """Bytes of one (padded) row of a split-embedding table (InterpreterNodes.cpp:43-74)."""
    so = 4 if scale_offset_is_fp32 else 2
    raw = {EST_FLOAT: num_dims * 4, EST_FLOAT16: num_dims * 2, EST_INT8: num_dims + 2 * so,
           EST_INT4: num_dims // 2 + 2 * so}[weights_ty]
    return (raw + row_alignment - 1) // row_alignment * row_alignment


def int_nbit_split_embedding_bags(dev_weights, uvm_weights, weights_placements, weights_offsets, weights_tys,
                                  dim_offsets, total_dims, indices, offsets, pooling_mode=EP_SUM, *,
                                  indice_weights=None, out_dtype=torch.float32, scale_offset_is_fp32=False,
                                  row_alignment=16, out=None, status=None):
    """IntNBitSplitEmbeddingBags (indice_weights None) / IntNBitSplitEmbeddingWeightedBags:
    T tables in one byte buffer, T*B bags per request, result [B, total_dims]."""
    _cuda(dev_weights, "dev_weights", (torch.uint8,))
    _cuda(uvm_weights, "uvm_weights", (torch.uint8,))
    _cuda(weights_placements, "weights_placements", (torch.int32,))
    _cuda(weights_offsets, "weights_offsets", (torch.int32, torch.int64))
    _cuda(weights_tys, "weights_tys", (torch.uint8,))
    _cuda(dim_offsets, "dim_offsets", (torch.int32,))
    _cuda(indices, "indices", (torch.int32, torch.int64))
    _cuda(offsets, "offsets", (indices.dtype,))
    if indice_weights is not None:
        _cuda(indice_weights, "indice_weights", (torch.float32, torch.float16))
    T = dim_offsets.shape[0] - 1
    if T < 0 or weights_tys.shape[0] != T or weights_placements.shape[0] != T or weights_offsets.shape[0] != T:
        raise ValueError("table description arrays disagree on the number of tables")
    if T == 0 or (offsets.shape[0] - 1) % T != 0:
        raise ValueError("offsets must hold num_tables * bags_per_table + 1 entries")
    B = (offsets.shape[0] - 1) // T
    if out is None:
        out = torch.empty((B, total_dims), dtype=out_dtype, device=indices.device)
    _cuda(out, "out", (torch.float32, torch.float16))
    check(_lib.lib().glowb200_int_nbit_split_embedding_bags(
        _p(out), _p(dev_weights), dev_weights.numel(), _p(uvm_weights), uvm_weights.numel(), _p(weights_placements),
        _p(weights_offsets), int(weights_offsets.dtype == torch.int64), _p(weights_tys), _p(dim_offsets), T,
        total_dims, _p(indices), _p(offsets), int(indices.dtype == torch.int64), indices.shape[0], B, pooling_mode,
        _p(indice_weights), int(indice_weights is not None and indice_weights.dtype == torch.float16),
        int(out.dtype == torch.float16), int(scale_offset_is_fp32), row_alignment, _p(status), _stream()))
    return out


# ------------------------------------------------------------------------------------------
# Int8 dense layers
# ------------------------------------------------------------------------------------------
FC_WEIGHT_OFFSETS_ZERO = 1
FC_FORCE_ANY_SHAPE_KERNEL = 2
FC_FUSE_RELU = 4
FC_BIAS_INT8 = 8

ASYMMETRIC, SYMMETRIC, SYMMETRIC_WITH_UNSIGNED, SYMMETRIC_WITH_POWER2_SCALE = 0, 1, 2, 3


def sparse_lengths_weighted_sum(data, weights, indices, lengths, *, out=None, status=None, workspace=None,
                                num_indices=None):
    """SparseLengthsWeightedSum over an fp32 table [rows, D]; weights=None is SparseLengthsSum."""
    _cuda(data, "data", (torch.float32,))
    _cuda(indices, "indices", (torch.int32, torch.int64))
    _cuda(lengths, "lengths", (torch.int32,))
    if weights is not None:
        _cuda(weights, "weights", (torch.float32,))
    rows, line = data.shape
    segments = lengths.shape[0]
    if out is None:
        out = torch.empty((segments, line), dtype=torch.float32, device=data.device)
    n = indices.shape[0] if num_indices is None else int(num_indices)
    ws = _workspace(workspace, slws_workspace_bytes(segments, 1), data.device)
    check(_lib.lib().glowb200_sparse_lengths_weighted_sum_f32(
        _p(out), _p(data), rows, _p(weights), _p(indices), int(indices.dtype == torch.int64), _p(lengths), segments, n,
        line, _p(ws), ws.numel(), _p(status), _stream()))
    return out


def sparse_lengths_sum(data, indices, lengths, **kw):
    return sparse_lengths_weighted_sum(data, None, indices, lengths, **kw)


def rowwise_quantized_sparse_lengths_weighted_sum(data, scales, offsets, weights, indices, lengths, *, out=None,
                                                  status=None, workspace=None, num_indices=None):
    """RowwiseQuantizedSparseLengthsWeightedSum: uint8 table [rows, D] with fp32 scales/offsets [rows]."""
    _cuda(data, "data", (torch.uint8,))
    _cuda(scales, "scales", (torch.float32,))
    _cuda(offsets, "offsets", (torch.float32,))
    _cuda(weights, "weights", (torch.float32,))
    _cuda(indices, "indices", (torch.int32, torch.int64))
    _cuda(lengths, "lengths", (torch.int32,))
    rows, line = data.shape
    segments = lengths.shape[0]
    if out is None:
        out = torch.empty((segments, line), dtype=torch.float32, device=data.device)
    n = indices.shape[0] if num_indices is None else int(num_indices)
    ws = _workspace(workspace, slws_workspace_bytes(segments, 1), data.device)
    check(_lib.lib().glowb200_rowwise_quantized_sparse_lengths_weighted_sum_f32(
        _p(out), _p(data), _p(scales), _p(offsets), rows, _p(weights), _p(indices),
        int(indices.dtype == torch.int64), _p(lengths), segments, n, line, _p(ws), ws.numel(), _p(status), _stream()))
    return out


def fused_row_bytes(cols, kind):
    """Row width in bytes of a fused-rowwise table of `cols` columns."""
    return (cols // 2 if kind in (UINT4_FUSED, UINT4_FUSED_FP16) else cols) + (4 if kind in (UINT8_FUSED_FP16, UINT4_FUSED_FP16) else 8)


def fused_rowwise_quantize_host(table, kind=UINT8_FUSED):
    """Host fused-rowwise quantisation of a float32 numpy matrix -> uint8 numpy [rows, row bytes]."""
    import numpy as np
    table = np.ascontiguousarray(table, np.float32)
    rows, cols = table.shape
    out = np.empty((rows, fused_row_bytes(cols, kind)), np.uint8)
    check(_lib.lib().glowb200_fused_rowwise_quantize(C.c_void_p(table.ctypes.data), rows, cols, int(kind),
                                                     C.c_void_p(out.ctypes.data), out.shape[1]))
    return out


def fused_rowwise_quantize(table, kind=UINT8_FUSED, out=None):
    """Fused-rowwise quantisation of a CUDA float32 matrix on the device."""
    _cuda(table, "table", (torch.float32,))
    rows, cols = table.shape
    if out is None:
        out = torch.empty((rows, fused_row_bytes(cols, kind)), dtype=torch.uint8, device=table.device)
    check(_lib.lib().glowb200_fused_rowwise_quantize_device(_p(table), rows, cols, int(kind), _p(out), out.shape[1],
                                                            _stream()))
    return out


def pad_fused_rows(table, kind, row_bytes, out=None):
    """A fused-rowwise CUDA table [rows, in_line] with every row padded to `row_bytes`: payload
    first, zeros, scale/offset as the last bytes.  The gather-pool operators take the padded table
    with out_line = the original column count and give bit-identical results; rows that fill whole
    128-byte lines cost one DRAM access each instead of one and a half."""
    _cuda(table, "table", (torch.uint8,))
    rows, in_line = table.shape
    tail = 4 if kind & 1 else 8
    if out is None:
        out = torch.empty((rows, row_bytes), dtype=torch.uint8, device=table.device)
    check(_lib.lib().glowb200_fused_rows_pad(_p(table), rows, in_line, tail, _p(out), row_bytes, _stream()))
    return out


def sum_partials(partials, out_dtype=torch.float32, out=None):
    """Sum of fp32 partial results [num, ...] over the first axis, cast once to out_dtype."""
    _cuda(partials, "partials", (torch.float32,))
    num = partials.shape[0]
    n = partials[0].numel()
    if out is None:
        out = torch.empty(partials.shape[1:], dtype=out_dtype, device=partials.device)
    check(_lib.lib().glowb200_sum_partials(_p(partials), num, partials.stride(0), n, _p(out),
                                           int(out.dtype == torch.float16), _stream()))
    return out


def choose_quantization_params(mn, mx, schema=ASYMMETRIC, bits=8):
    """(scale, offset) for a float range -- host computation (chooseQuantizationParams)."""
    sc, off = C.c_float(), C.c_int32()
    _lib.lib().glowb200_choose_quantization_params(C.c_float(float(mn)), C.c_float(float(mx)), int(schema), int(bits),
                                                   C.byref(sc), C.byref(off))
    return float(sc.value), int(off.value)


def tensor_rowwise_quantize_i8(w, schema=ASYMMETRIC):
    """Host rowwise quantisation of a float32 numpy matrix -> (int8, scales, offsets) numpy arrays."""
    import numpy as np
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    q, sc, off = np.empty((rows, cols), np.int8), np.empty(rows, np.float32), np.empty(rows, np.int32)
    check(_lib.lib().glowb200_tensor_rowwise_quantize_i8(C.c_void_p(w.ctypes.data), rows, cols, int(schema),
                                                         C.c_void_p(q.ctypes.data), C.c_void_p(sc.ctypes.data),
                                                         C.c_void_p(off.ctypes.data)))
    return q, sc, off


def channelwise_conv_prepare(filt, bias, in_scale, schema=SYMMETRIC):
    """Host preparation of a channelwise-quantized convolution's constants from a float filter
    [outC, kH, kW, inC/group] and float bias [outC] (numpy).  Returns a dict of numpy arrays:
    filter (int8, same shape), filter_scales, filter_offsets, bias (int32), bias_scales, bias_offsets."""
    import numpy as np
    filt = np.ascontiguousarray(filt, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    oc = filt.shape[0]
    k = filt.size // oc
    out = dict(filter=np.empty(filt.shape, np.int8), filter_scales=np.empty(oc, np.float32),
               filter_offsets=np.empty(oc, np.int32), bias=np.empty(oc, np.int32),
               bias_scales=np.empty(oc, np.float32), bias_offsets=np.empty(oc, np.int32))
    check(_lib.lib().glowb200_channelwise_conv_prepare(
        C.c_void_p(filt.ctypes.data), C.c_void_p(bias.ctypes.data), oc, k, C.c_float(float(in_scale)), int(schema),
        *[C.c_void_p(out[n].ctypes.data) for n in ("filter", "filter_scales", "filter_offsets", "bias", "bias_scales",
                                                  "bias_offsets")]))
    return out


def quantize_bias_i32(b, scale, offset=0):
    import numpy as np
    b = np.ascontiguousarray(b, np.float32)
    out = np.empty(b.shape, np.int32)
    check(_lib.lib().glowb200_quantize_bias_i32(C.c_void_p(b.ctypes.data), b.size, C.c_float(float(scale)), int(offset),
                                                C.c_void_p(out.ctypes.data)))
    return out


def quantize_scale_offset_32to8(scale):
    """(pre, post, integer scale) for a float rescale factor -- host computation."""
    out = (C.c_int32 * 3)()
    base = C.addressof(out)
    _lib.lib().glowb200_quantize_scale_offset_32to8(C.c_float(float(scale)), C.c_void_p(base), C.c_void_p(base + 4),
                                                    C.c_void_p(base + 8))
    return int(out[0]), int(out[1]), int(out[2])


def rowwise_requant_params(row_scales, in_scale, bias_scales, out_scale):
    """Host derivation of (bias_pre, bias_post, bias_scale, out_pre, out_post, out_scale) int32
    numpy arrays for a rowwise FC / channelwise conv."""
    import numpy as np
    rs = np.ascontiguousarray(row_scales, np.float32)
    bs = np.ascontiguousarray(np.atleast_1d(bias_scales), np.float32)
    outs = [np.empty(rs.shape[0], np.int32) for _ in range(6)]
    check(_lib.lib().glowb200_rowwise_requant_params(
        C.c_void_p(rs.ctypes.data), rs.shape[0], C.c_float(float(in_scale)), C.c_void_p(bs.ctypes.data),
        bs.shape[0], C.c_float(float(out_scale)), *[C.c_void_p(o.ctypes.data) for o in outs]))
    return outs


def wait_limit_selftest(limit_cycles, status):
    """Runs the library's bounded device-side wait on a barrier nothing completes; returns how
    many of the two waiting warps gave up (the status word gets STATUS_WAIT_TIMEOUT)."""
    gave_up = torch.zeros(1, dtype=torch.int32, device=status.device)
    check(_lib.lib().glowb200_wait_limit_selftest(int(limit_cycles), _p(status), _p(gave_up), _stream()))
    return gave_up


def i8_mma_issue_rate(mmas_per_sm=32768, repeats=4, status=None):
    """TOP/s of the tensor pipe issuing int8 MMAs on resident tiles (best of `repeats` launches,
    device-timed): the measured ceiling an int8 contraction is compared with."""
    ops_out = C.c_int64(0)
    best = 0.0
    for i in range(repeats + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(_lib.lib().glowb200_i8_mma_issue_probe(int(mmas_per_sm), C.byref(ops_out), _p(status), _stream()))
        e1.record()
        e1.synchronize()
        if i:  # the first launch warms up
            best = max(best, ops_out.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def i8_gemm_workspace_bytes(M, K, N):
    return int(_lib.lib().glowb200_i8_gemm_workspace_bytes(int(M), int(K), int(N)))


def i8_row_sums(matrix):
    _cuda(matrix, "matrix", (torch.int8,))
    out = torch.empty(matrix.shape[0], dtype=torch.int32, device=matrix.device)
    check(_lib.lib().glowb200_i8_row_sums(_p(matrix), matrix.shape[0], matrix.shape[1], _p(out), _stream()))
    return out


def rowwise_quantized_fc(inp, weights, bias, weights_offsets, bias_triples, out_triples, out_offset, in_offset,
                         bias_offset, *, weights_row_sums=None, flags=0, out=None, workspace=None, status=None):
    """RowwiseQuantizedFullyConnected: inp int8 [M,K], weights int8 [N,K], bias int32 [N],
    weights_offsets int32 [N], bias_triples/out_triples = three int32 [N] tensors each."""
    _cuda(inp, "inp", (torch.int8,))
    _cuda(weights, "weights", (torch.int8,))
    M, K = inp.shape
    N = weights.shape[0]
    _cuda(bias, "bias", (torch.int32, torch.int8))
    if bias.dtype == torch.int8:   # the reference's _i8_i8 form
        flags |= FC_BIAS_INT8
    for t in (weights_offsets, *bias_triples, *out_triples):
        _cuda(t, "per-row parameter", (torch.int32,))
    if out is None:
        out = torch.empty((M, N), dtype=torch.int8, device=inp.device)
    ws = _workspace(workspace, i8_gemm_workspace_bytes(M, K, N), inp.device)
    check(_lib.lib().glowb200_rowwise_quantized_fc_i8_i32(
        _p(out), _p(inp), _p(weights), _p(bias), _p(weights_offsets), _p(bias_triples[0]), _p(bias_triples[1]),
        _p(bias_triples[2]), _p(out_triples[0]), _p(out_triples[1]), _p(out_triples[2]), M, K, N, int(out_offset),
        int(in_offset), int(bias_offset), _p(weights_row_sums), int(flags), _p(ws), ws.numel(), _p(status),
        _stream()))
    return out


def fully_connected_i8(inp, weights, bias, out_offset, in_offset, weights_offset, bias_offset, bias_triple,
                       out_triple, *, weights_transposed=None, flags=0, out=None, workspace=None, status=None):
    """FullyConnected (int8, per-tensor): inp [M,K], weights [K,N], bias int32 (or int8) [N]."""
    if bias.dtype == torch.int8:   # the reference's _i8_i8 form
        flags |= FC_BIAS_INT8
    M, K = inp.shape
    N = weights.shape[1] if weights is not None else weights_transposed.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.int8, device=inp.device)
    ws = _workspace(workspace, i8_gemm_workspace_bytes(M, K, N), inp.device)
    check(_lib.lib().glowb200_fc_i8_i32(
        _p(out), _p(inp), _p(weights), _p(bias), M, K, N, int(out_offset), int(in_offset), int(weights_offset),
        int(bias_offset), *[int(v) for v in bias_triple], *[int(v) for v in out_triple], _p(weights_transposed),
        int(flags), _p(ws), ws.numel(), _p(status), _stream()))
    return out


def matmul_i8(lhs, rhs, out_offset, lhs_offset, rhs_offset, out_triple, *, flags=0, out=None, workspace=None,
              status=None):
    """MatMul (int8): lhs [M,K], rhs [K,N]."""
    M, K = lhs.shape
    N = rhs.shape[1]
    if out is None:
        out = torch.empty((M, N), dtype=torch.int8, device=lhs.device)
    ws = _workspace(workspace, i8_gemm_workspace_bytes(M, K, N), lhs.device)
    check(_lib.lib().glowb200_matmul_i8(
        _p(out), _p(lhs), _p(rhs), M, K, N, int(out_offset), int(lhs_offset), int(rhs_offset),
        *[int(v) for v in out_triple], int(flags), _p(ws), ws.numel(), _p(status), _stream()))
    return out


def tensor_rowwise_quantize_i8_device(w, schema=ASYMMETRIC):
    """tensorRowwiseQuantization on the device: fp32 [rows, cols] -> (int8, scales fp32, offsets int32)."""
    _cuda(w, "w", (torch.float32,))
    rows, cols = w.shape
    q = torch.empty((rows, cols), dtype=torch.int8, device=w.device)
    scales = torch.empty(rows, dtype=torch.float32, device=w.device)
    offsets = torch.empty(rows, dtype=torch.int32, device=w.device)
    check(_lib.lib().glowb200_tensor_rowwise_quantize_i8_device(_p(w), rows, cols, schema, _p(q), _p(scales), _p(offsets),
                                                                _stream()))
    return q, scales, offsets


def quantize_rows_i8_device(w, scales, offsets):
    """fp32 [rows, cols] quantized with given per-row parameters."""
    _cuda(w, "w", (torch.float32,))
    rows, cols = w.shape
    q = torch.empty((rows, cols), dtype=torch.int8, device=w.device)
    check(_lib.lib().glowb200_quantize_rows_i8_device(_p(w), rows, cols, _p(scales), _p(offsets), _p(q), _stream()))
    return q


def quantization_profile(x, comp_info, histogram, *, workspace=None):
    """QuantizationProfile: folds tensor x into the running {min, max} (comp_info, 2 floats) and the
    running histogram, both updated in place on the device."""
    _cuda(x, "x", (torch.float32,))
    _cuda(comp_info, "comp_info", (torch.float32,))
    _cuda(histogram, "histogram", (torch.float32,))
    bins = histogram.numel()
    ws = _workspace(workspace, int(_lib.lib().glowb200_quantization_profile_workspace_bytes(bins)), x.device)
    check(_lib.lib().glowb200_quantization_profile(_p(x), x.numel(), _p(comp_info), _p(histogram), bins, _p(ws),
                                                   ws.numel(), _stream()))
    return comp_info, histogram


def dynamic_fc_workspace_bytes(M, K, N):
    return int(_lib.lib().glowb200_dynamic_fc_workspace_bytes(M, K, N))


def dynamic_rowwise_quantized_fc(inp, weights, bias, scales, offsets, *, weights_transposed=None, flags=0, out=None,
                                 workspace=None, status=None):
    """DynamicRowwiseQuantizedFullyConnected: inp [M,K] fp16, weights [K,N] int8 (or weights_transposed
    [N,K]), bias / scales fp32 [N], offsets int32 [N]; result [M,N] fp16."""
    _cuda(inp, "inp", (torch.float16,))
    M, K = inp.shape
    N = bias.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=inp.device)
    ws = _workspace(workspace, dynamic_fc_workspace_bytes(M, K, N), inp.device)
    check(_lib.lib().glowb200_dynamic_rowwise_quantized_fc(
        _p(out), _p(inp), _p(weights), _p(bias), _p(scales), _p(offsets), M, K, N, _p(weights_transposed), int(flags),
        _p(ws), ws.numel(), _p(status), _stream()))
    return out


def dynamic_quantized_fc(inp, weights, bias, weights_scale, weights_offset, *, weights_transposed=None, flags=0,
                         out=None, workspace=None, status=None):
    """DynamicQuantizedFullyConnected: as above with one scale / offset for the whole weights tensor."""
    _cuda(inp, "inp", (torch.float16,))
    M, K = inp.shape
    N = bias.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=inp.device)
    ws = _workspace(workspace, dynamic_fc_workspace_bytes(M, K, N), inp.device)
    check(_lib.lib().glowb200_dynamic_quantized_fc(
        _p(out), _p(inp), _p(weights), _p(bias), float(weights_scale), int(weights_offset), M, K, N,
        _p(weights_transposed), int(flags), _p(ws), ws.numel(), _p(status), _stream()))
    return out


# ------------------------------------------------------------------------------------------
# Int8 convolution and glue operators
# ------------------------------------------------------------------------------------------
def _i64arr(v):
    return (C.c_int64 * len(v))(*[int(x) for x in v])


def conv_out_hw(in_hw, kernels, strides, pads, dilation=(1, 1)):
    """Output height/width as Glow computes them (calculateConvPoolOutputDims)."""
    oh = (in_hw[0] + pads[0] + pads[2] - ((kernels[0] - 1) * dilation[0] + 1)) // strides[0] + 1
    ow = (in_hw[1] + pads[1] + pads[3] - ((kernels[1] - 1) * dilation[1] + 1)) // strides[1] + 1
    return oh, ow


def _conv_shapes(inp, filt, kernels, strides, pads, group, dilation):
    n, h, w, c = inp.shape
    oc = filt.shape[0]
    oh, ow = conv_out_hw((h, w), kernels, strides, pads, dilation)
    return (_i64arr((n, oh, ow, oc)), _i64arr(inp.shape), _i64arr(filt.shape), _i64arr(kernels), _i64arr(strides),
            _i64arr(pads), int(group), _i64arr(dilation)), (n, oh, ow, oc)


def channelwise_quantized_conv2d(inp, filt, bias, kernels, strides, pads, group, dilation, out_offset, in_offset,
                                 filter_offsets, bias_offsets, bias_triples, out_triples, act_type=0, act_args=None,
                                 *, filter_row_sums=None, flags=0, out=None, workspace=None, status=None):
    """ChannelwiseQuantizedConvolution: inp int8 NHWC, filt int8 [outC,kH,kW,inC/group], bias int32."""
    _cuda(inp, "inp", (torch.int8,))
    _cuda(filt, "filt", (torch.int8,))
    sh, odims = _conv_shapes(inp, filt, kernels, strides, pads, group, dilation)
    if out is None:
        out = torch.empty(odims, dtype=torch.int8, device=inp.device)
    need = int(_lib.lib().glowb200_conv2d_workspace_bytes(sh[0], sh[1], sh[2], sh[3], sh[4], sh[5], sh[6], sh[7]))
    ws = _workspace(workspace, need, inp.device)
    aa = (C.c_int32 * 3)(*([int(v) for v in act_args] + [0, 0, 0])[:3]) if act_args is not None else None
    check(_lib.lib().glowb200_channelwise_quantized_conv2d_i8_i32(
        _p(out), _p(inp), _p(filt), _p(bias), sh[0], sh[1], sh[2], sh[3], sh[4], sh[5], sh[6], sh[7], int(out_offset),
        int(in_offset), _p(filter_offsets), _p(bias_offsets), _p(bias_triples[0]), _p(bias_triples[1]),
        _p(bias_triples[2]), _p(out_triples[0]), _p(out_triples[1]), _p(out_triples[2]), int(act_type), aa,
        _p(filter_row_sums), int(flags), _p(ws), ws.numel(), _p(status), _stream()))
    return out


def conv2d_i8(inp, filt, bias, kernels, strides, pads, group, dilation, out_offset, in_offset, filter_offset,
              bias_offset, bias_triple, out_triple, act_type=0, act_args=None, *, flags=0, out=None, workspace=None,
              status=None):
    """Convolution (int8, per-tensor quantisation)."""
    sh, odims = _conv_shapes(inp, filt, kernels, strides, pads, group, dilation)
    if out is None:
        out = torch.empty(odims, dtype=torch.int8, device=inp.device)
    need = int(_lib.lib().glowb200_conv2d_workspace_bytes(sh[0], sh[1], sh[2], sh[3], sh[4], sh[5], sh[6], sh[7]))
    ws = _workspace(workspace, need, inp.device)
    aa = (C.c_int32 * 3)(*([int(v) for v in act_args] + [0, 0, 0])[:3]) if act_args is not None else None
    check(_lib.lib().glowb200_conv2d_i8_i32(
        _p(out), _p(inp), _p(filt), _p(bias), sh[0], sh[1], sh[2], sh[3], sh[4], sh[5], sh[6], int(out_offset),
        int(in_offset), int(filter_offset), int(bias_offset), *[int(v) for v in bias_triple],
        *[int(v) for v in out_triple], sh[7], int(act_type), aa, int(flags), _p(ws), ws.numel(), _p(status), _stream()))
    return out


def element_add_i8(lhs, rhs, dest_offset, lhs_offset, rhs_offset, lhs_triple, rhs_triple, out=None):
    out = torch.empty_like(lhs) if out is None else out
    check(_lib.lib().glowb200_element_add_i8(_p(out), _p(lhs), _p(rhs), lhs.numel(), int(dest_offset), int(lhs_offset),
                                             int(rhs_offset), *[int(v) for v in lhs_triple],
                                             *[int(v) for v in rhs_triple], _stream()))
    return out


BINARY_ADD, BINARY_SUB, BINARY_MAX, BINARY_MIN = 0, 1, 2, 3


def element_binary_i8(op, lhs, rhs, dest_offset, lhs_offset, rhs_offset, lhs_triple, rhs_triple, out=None):
    """ElementAdd / Sub / Max / Min on int8 tensors (op: BINARY_*)."""
    out = torch.empty_like(lhs) if out is None else out
    check(_lib.lib().glowb200_element_binary_i8(int(op), _p(out), _p(lhs), _p(rhs), lhs.numel(), int(dest_offset),
                                                int(lhs_offset), int(rhs_offset), *[int(v) for v in lhs_triple],
                                                *[int(v) for v in rhs_triple], _stream()))
    return out


def element_muldiv_i8(is_div, lhs, rhs, dest_offset, lhs_offset, rhs_offset, triple, out=None):
    """ElementMul (is_div False) / ElementDiv (True) on int8 tensors."""
    out = torch.empty_like(lhs) if out is None else out
    check(_lib.lib().glowb200_element_muldiv_i8(int(bool(is_div)), _p(out), _p(lhs), _p(rhs), lhs.numel(), int(dest_offset),
                                                int(lhs_offset), int(rhs_offset), *[int(v) for v in triple], _stream()))
    return out


def batched_add_i8(batch, slice_, dest_offset, batch_offset, slice_offset, batch_triple, slice_triple, out=None):
    """BatchedAdd: slice_ (int8 or int32, [slice_size]) added to every row of batch [num_slices, slice_size]."""
    out = torch.empty_like(batch) if out is None else out
    num_slices = batch.shape[0]
    slice_size = batch.numel() // max(num_slices, 1)
    check(_lib.lib().glowb200_batched_add_i8(_p(out), _p(batch), _p(slice_), int(slice_.dtype == torch.int32), num_slices,
                                             slice_size, int(dest_offset), int(batch_offset), int(slice_offset),
                                             *[int(v) for v in batch_triple], *[int(v) for v in slice_triple], _stream()))
    return out


def element_add_maxsplat_i8(lhs, rhs, dest_offset, lhs_offset, rhs_offset, lhs_triple, rhs_triple, splat, out=None):
    """element_add_i8 followed by element_maxsplat_i8(splat), fused."""
    if out is None:
        out = torch.empty_like(lhs)
    check(_lib.lib().glowb200_element_add_maxsplat_i8(
        _p(out), _p(lhs), _p(rhs), lhs.numel(), int(dest_offset), int(lhs_offset), int(rhs_offset),
        *[int(v) for v in lhs_triple], *[int(v) for v in rhs_triple], int(splat), _stream()))
    return out


def element_relu_i8(src, src_offset, dest_offset, triple, out=None):
    out = torch.empty_like(src) if out is None else out
    check(_lib.lib().glowb200_element_relu_i8(_p(out), _p(src), src.numel(), int(src_offset), int(dest_offset),
                                              *[int(v) for v in triple], _stream()))
    return out


def element_maxsplat_i8(src, splat, out=None):
    out = torch.empty_like(src) if out is None else out
    check(_lib.lib().glowb200_element_maxsplat_i8(_p(out), _p(src), src.numel(), int(splat), _stream()))
    return out


def element_rescale_i8(src, out_offset, in_offset, triple, out=None):
    out = torch.empty_like(src) if out is None else out
    check(_lib.lib().glowb200_element_rescale_i8(_p(out), _p(src), src.numel(), int(out_offset), int(in_offset),
                                                 *[int(v) for v in triple], _stream()))
    return out


def element_quantize_i8(src, scale, offset, out=None):
    out = torch.empty(src.shape, dtype=torch.int8, device=src.device) if out is None else out
    check(_lib.lib().glowb200_element_quantize_i8(_p(out), _p(src), src.numel(), C.c_float(float(scale)), int(offset),
                                                  _stream()))
    return out


def element_dequantize_i8(src, scale, offset, out=None):
    out = torch.empty(src.shape, dtype=torch.float32, device=src.device) if out is None else out
    check(_lib.lib().glowb200_element_dequantize_i8(_p(out), _p(src), src.numel(), C.c_float(float(scale)),
                                                    int(offset), _stream()))
    return out


def max_pool_i8(inp, kernels, strides, pads, out_offset, out=None):
    n, h, w, c = inp.shape
    oh, ow = conv_out_hw((h, w), kernels, strides, pads)
    out = torch.empty((n, oh, ow, c), dtype=torch.int8, device=inp.device) if out is None else out
    check(_lib.lib().glowb200_max_pool_i8(_p(inp), _p(out), _i64arr(inp.shape), _i64arr(out.shape), _i64arr(kernels),
                                          _i64arr(strides), _i64arr(pads), int(out_offset), _stream()))
    return out


def avg_pool_i8(inp, kernels, strides, pads, count_include_pads, out_offset, in_offset, triple, out=None):
    n, h, w, c = inp.shape
    oh, ow = conv_out_hw((h, w), kernels, strides, pads)
    out = torch.empty((n, oh, ow, c), dtype=torch.int8, device=inp.device) if out is None else out
    check(_lib.lib().glowb200_avg_pool_i8(_p(inp), _p(out), _i64arr(inp.shape), _i64arr(out.shape), _i64arr(kernels),
                                          _i64arr(strides), _i64arr(pads), int(bool(count_include_pads)),
                                          int(out_offset), int(in_offset), *[int(v) for v in triple], _stream()))
    return out


def transpose(src, shuffle):
    """dest dims[i] = src dims[shuffle[i]] (NCHW -> NHWC is shuffle (0, 2, 3, 1))."""
    if src.element_size() not in (1, 4):
        raise TypeError("1- or 4-byte elements only")
    out = torch.empty([src.shape[i] for i in shuffle], dtype=src.dtype, device=src.device)
    check(_lib.lib().glowb200_transpose(_p(src), _p(out), _i64arr(src.shape), (C.c_int32 * len(shuffle))(*shuffle),
                                        len(shuffle), src.element_size(), _stream()))
    return out


class programmatic_launch:
    """with programmatic_launch(False): ...  -- ordinary launches inside (e.g. for a stream that runs
    beside another one); the previous setting comes back on exit."""

    def __init__(self, enabled):
        self.enabled = enabled

    def __enter__(self):
        self.before = _lib.lib().glowb200_set_programmatic_launch(1 if self.enabled else 0)
        return self

    def __exit__(self, *exc):
        _lib.lib().glowb200_set_programmatic_launch(self.before)
        return False


def quantize_transpose_i8(src, shuffle, scale, offset):
    """transpose(quantize(src)) in one pass: fp32 in, int8 out with dims[i] = src dims[shuffle[i]]."""
    _cuda(src, "src", (torch.float32,))
    out = torch.empty([src.shape[i] for i in shuffle], dtype=torch.int8, device=src.device)
    check(_lib.lib().glowb200_quantize_transpose_i8(_p(out), _p(src), _i64arr(src.shape), (C.c_int32 * len(shuffle))(*shuffle),
                                                    len(shuffle), C.c_float(float(scale)), int(offset), _stream()))
    return out


def pairwise_dot_interaction(dense, pooled, *, quant=None, out=None):
    """dense fp32 [B, D]; pooled fp32 [B, T, D] (or [B, T*D]).  Returns fp32 [B, D + n(n-1)/2]
    (n = T + 1), or int8 when quant=(scale, offset) (the following Quantize node fused)."""
    _cuda(dense, "dense", (torch.float32,))
    _cuda(pooled, "pooled", (torch.float32,))
    B, D = dense.shape
    T = pooled.numel() // (B * D) if B else 0
    n = T + 1
    width = D + n * (n - 1) // 2
    if out is None:
        out = torch.empty((B, width), dtype=torch.int8 if quant else torch.float32, device=dense.device)
    q = quant or (1.0, 0)
    check(_lib.lib().glowb200_pairwise_dot_interaction(
        _p(dense), D, _p(pooled), T * D, B, T, D, None if quant else _p(out), _p(out) if quant else None, width,
        C.c_float(float(q[0])), int(q[1]), _stream()))
    return out


def device_tensor(ptr, shape, dtype, device="cuda"):
    """A torch view (no copy) of device memory the library owns -- a placeholder of a loaded
    network (DeviceManager.placeholder_address), for device-resident tensors."""
    class _Raw:
        pass
    raw = _Raw()
    typestr = {torch.float32: "<f4", torch.uint8: "|u1", torch.int8: "|i1", torch.float16: "<f2", torch.int32: "<i4",
               torch.int64: "<i8"}[dtype]
    raw.__cuda_array_interface__ = {"shape": tuple(int(v) for v in shape), "typestr": typestr, "data": (int(ptr), False),
                                    "version": 3}
    return torch.as_tensor(raw, device=device)


class PeerBuffer:
    """Device memory the other GPUs of the node can store into (set-up time object).
    `handle` (64 bytes) is what the owning process sends to its peers; `open` maps a peer's."""

    def __init__(self, nbytes):
        ptr = C.c_void_p()
        h = (C.c_ubyte * 64)()
        check(_lib.lib().glowb200_peer_buffer_create(int(nbytes), C.byref(ptr), h))
        self.ptr, self.nbytes, self.handle = int(ptr.value), int(nbytes), bytes(h)
        self._opened = []

    def open(self, handle):
        ptr = C.c_void_p()
        buf = (C.c_ubyte * 64).from_buffer_copy(handle)
        check(_lib.lib().glowb200_peer_buffer_open(buf, C.byref(ptr)))
        self._opened.append(int(ptr.value))
        return int(ptr.value)

    def as_tensor(self, shape, dtype):
        """A torch view of the local buffer (no copy)."""
        class _Raw:
            pass
        raw = _Raw()
        typestr = {torch.float32: "<f4", torch.uint8: "|u1", torch.int8: "|i1", torch.float16: "<f2"}[dtype]
        raw.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (self.ptr, False), "version": 3}
        return torch.as_tensor(raw, device="cuda")

    def release(self):
        for p in self._opened:
            _lib.lib().glowb200_peer_buffer_close(C.c_void_p(p))
        self._opened = []
        if self.ptr:
            _lib.lib().glowb200_peer_buffer_destroy(C.c_void_p(self.ptr))
            self.ptr = 0


def peer_rendezvous(my_flags_ptr, peer_ptrs_dev, world, rank, status=None, limit_cycles=4_000_000_000):
    """One rendezvous of the ranks whose flag buffers are listed in the device array
    `peer_ptrs_dev` (int64 tensor of `world` addresses); see glowb200_peer_rendezvous."""
    check(_lib.lib().glowb200_peer_rendezvous(C.c_void_p(int(my_flags_ptr)), _p(peer_ptrs_dev), int(world), int(rank),
                                              int(limit_cycles), _p(status), _stream()))


class SlwsBatch:
    """A fixed set of tables of one kind and row width, pooled by ONE launch per request.

    The descriptor array lives on the device; `bind` rewrites it (one small H2D copy) when the
    request buffers move, `run` launches.  dest_stride / dest pointers may address slices of a
    wider [segments, tables * D] buffer so the tables' results land concatenated.
    """

    def __init__(self, kind, in_line, index_dtype=torch.int64, use_fp16_accumulation=False, device="cuda",
                 out_line=None):
        self.kind, self.in_line = kind, in_line
        self.out_line = out_columns(in_line, kind) if out_line is None else int(out_line)
        self.index_dtype = index_dtype
        self.fp16_acc = use_fp16_accumulation
        self.device = torch.device(device)
        self.jobs_dev = None
        self.sharded = False
        self.num_jobs = 0
        self.max_segments = 0
        self.workspace = None
        self._keep = None

    def bind(self, tables, weights, indices, lengths, dests, dest_stride=None, scatter=None, bags_per_dest=0,
             row_ranges=None):
        """scatter: optional list (one entry per table) of lists of destination base addresses
        (ints, possibly in other GPUs' memory); bag b of table i then goes to row
        b % bags_per_dest of scatter[i][b // bags_per_dest].
        row_ranges: optional list (one entry per table) of (row_begin, global_rows) for tables
        that are row-range shards: indices then number the whole table, and rows of other shards
        are skipped, so the result is this shard's partial sum."""
        n = len(tables)
        arr = (SlwsJob * n)()
        odt = result_dtype(self.kind)
        self.max_segments = 0
        for i in range(n):
            _cuda(tables[i], "table", (torch.uint8,))
            _cuda(weights[i], "weights", (odt, torch.float16, torch.float32))
            _cuda(indices[i], "indices", (self.index_dtype,))
            _cuda(lengths[i], "lengths", (torch.int32,))
            if tables[i].shape[1] != self.in_line:
                raise ValueError("all tables of a batch share one row width")
            # the batched kernels use vector loads on the strength of these alignments
            for what, ten, al in (("table", tables[i], 16), ("weights", weights[i], weights[i].element_size()),
                                  ("indices", indices[i], indices[i].element_size()), ("lengths", lengths[i], 4)):
                if ten.data_ptr() % al:
                    raise ValueError("%s %d of a batched launch must start on a %d-byte boundary" % (what, i, al))
            j = arr[i]
            j.data, j.weights, j.indices = tables[i].data_ptr(), weights[i].data_ptr(), indices[i].data_ptr()
            j.lengths = lengths[i].data_ptr()
            j.dest = dests[i].data_ptr() if dests is not None else 0
            j.rows, j.num_indices = tables[i].shape[0], indices[i].shape[0]
            j.dest_stride = self.out_line if dest_stride is None else dest_stride
            j.segments = lengths[i].shape[0]
            if row_ranges is not None:
                j.row_begin, j.global_rows = int(row_ranges[i][0]), int(row_ranges[i][1])
            self.max_segments = max(self.max_segments, j.segments)
        self.sharded = row_ranges is not None
        self._scatter_dev = None
        if scatter is not None:
            per = len(scatter[0])
            flat = torch.tensor([a for row in scatter for a in row], dtype=torch.int64).to(self.device)
            self._scatter_dev = flat
            for i in range(n):
                arr[i].dests = flat.data_ptr() + 8 * per * i
                arr[i].bags_per_dest = int(bags_per_dest)
        self.out_fp16 = int(weights[0].dtype == torch.float16) if n else 0
        host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8) if n else torch.empty(0, dtype=torch.uint8)
        self.jobs_dev = host.to(self.device)
        self.num_jobs = n
        need = slws_workspace_bytes(self.max_segments, max(n, 1))
        if self.workspace is None or self.workspace.numel() < need:
            self.workspace = torch.empty(max(need, 8), dtype=torch.uint8, device=self.device)
        self._keep = (tables, weights, indices, lengths, dests)
        return self

    def run(self, status=None):
        if self.sharded:
            if self.out_fp16 or self.fp16_acc:
                raise ValueError("row-range shards take fp32 weights and give fp32 partial sums")
            check(_lib.lib().glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_row_sharded(
                _p(self.jobs_dev), self.num_jobs, self.max_segments, self.kind,
                int(self.index_dtype == torch.int64), self.in_line, self.out_line,
                _p(self.workspace), self.workspace.numel(), _p(status), _stream()))
            return
        check(_lib.lib().glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_batched(
            _p(self.jobs_dev), self.num_jobs, self.max_segments, self.kind,
            int(self.index_dtype == torch.int64), self.in_line, self.out_line, self.out_fp16, int(self.fp16_acc),
            _p(self.workspace), self.workspace.numel(), _p(status), _stream()))
