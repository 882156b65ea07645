"""TEST INFRASTRUCTURE ONLY -- not part of the product.

numpy/ctypes front end of the two CPU checkers:

* ``liboracle.so``  -- our plain-C restatement of the reference arithmetic
  (``oracle/glow_oracle.c``), always available after ``make -C oracle``.
* ``_ref/libjit_strict.so`` / ``_ref/libjit_fast.so`` -- pytorch/glow's own libjit kernel
  sources (lib/LLVMIRCodeGen/libjit/*.cpp) compiled unmodified; present when they were
  built on a machine that has the reference tree (the files then travel with the repo).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

KIND_U8_F32, KIND_U8_F16, KIND_U4_F32, KIND_U4_F16 = 0, 1, 2, 3

_i64, _i32, _f32, _vp = C.c_int64, C.c_int32, C.c_float, C.c_void_p


def reference_dir():
    """The checkout of pytorch/glow the reference libraries are compiled from: GLOW_REFERENCE_DIR,
    else the `reference` directory beside the repository, when either exists."""
    for d in (os.environ.get("GLOW_REFERENCE_DIR"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if d and os.path.exists(os.path.join(d, "lib", "LLVMIRCodeGen", "libjit", "libjit.cpp")):
            return d
    return ""


def build(with_ref=True):
    """Compile liboracle.so (and, where the reference tree exists, oracle/_ref)."""
    subprocess.check_call(["make", "-s", "-C", HERE, "all" if with_ref else HERE + "/liboracle.so",
                           "REF=" + (reference_dir() if with_ref else "")])


class _Ptr(C.c_void_p):
    """A void* argument that keeps the array it points into alive for the call."""


def _ptr(a):
    if a is None:
        return C.c_void_p(0)
    p = _Ptr(a.ctypes.data)
    p._keep = a
    return p


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build(with_ref=False)
        _lib = C.CDLL(path)
        _lib.orc_scale32.restype = _i32
        _lib.orc_scale32.argtypes = [_i32] * 5
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [_f32]
        _lib.orc_f16_to_f32.restype = _f32
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_quantize_scale_offset_32to8.argtypes = [_f32, _vp, _vp, _vp]
    return _lib


_ref = {}


def ref(flavour="strict"):
    """The reference's own libjit build, or None when it is not present."""
    if flavour not in _ref:
        path = os.path.join(HERE, "_ref", "libjit_%s.so" % flavour)
        _ref[flavour] = C.CDLL(path) if os.path.exists(path) else None
    return _ref[flavour]


def ref_available(flavour="strict"):
    return ref(flavour) is not None


# ---------------------------------------------------------------------------- scalars
def scale32(x, pre, post, scale, offset):
    return lib().orc_scale32(int(x), int(pre), int(post), int(scale), int(offset))


def quantize_scale_offset_32to8(scale):
    """-> (pre, post, integer scale) of quantizeScaleOffset32To8(scale, *)."""
    out = (C.c_int32 * 3)()
    base = C.addressof(out)
    lib().orc_quantize_scale_offset_32to8(C.c_float(float(np.float32(scale))), _vp(base), _vp(base + 4), _vp(base + 8))
    return int(out[0]), int(out[1]), int(out[2])


def rowwise_requant_params(w_scales, in_scale, bias_scales, out_scale):
    """Per-row (bias_pre, bias_post, bias_scale, out_pre, out_post, out_scale) int32 arrays."""
    ws = _c(w_scales, np.float32)
    bs = _c(np.atleast_1d(bias_scales), np.float32)
    n = ws.shape[0]
    outs = [np.empty(n, np.int32) for _ in range(6)]
    lib().orc_rowwise_requant_params(_ptr(ws), _i64(n), _f32(in_scale), _ptr(bs), _i64(bs.shape[0]),
                                     _f32(out_scale), *[_ptr(o) for o in outs])
    return outs


def f32_to_f16_bits(a):
    a = _c(a, np.float32).ravel()
    f = lib().orc_f32_to_f16
    return np.array([f(float(x)) for x in a], dtype=np.uint16)


def choose_quantization_params(mn, mx, schema=0, qmin=-128, qmax=127):
    """-> (scale float32, offset int) of chooseQuantizationParams without calibration."""
    sc, off = C.c_float(), C.c_int32()
    lib().orc_choose_quantization_params(_f32(float(np.float32(mn))), _f32(float(np.float32(mx))), C.c_int(schema),
                                         _i64(qmin), _i64(qmax), C.byref(sc), C.byref(off))
    return np.float32(sc.value), int(off.value)


def tensor_rowwise_quantize_i8(w, schema=0):
    """-> (int8 [rows, cols], float32 scales [rows], int32 offsets [rows])."""
    w = _c(w, np.float32)
    rows, cols = w.shape
    q, sc, off = np.empty((rows, cols), np.int8), np.empty(rows, np.float32), np.empty(rows, np.int32)
    lib().orc_tensor_rowwise_quantize_i8(_ptr(w), _i64(rows), _i64(cols), C.c_int(schema), _ptr(q), _ptr(sc), _ptr(off))
    return q, sc, off


# ---------------------------------------------------------------------------- tables
def fused_line_bytes(cols, kind):
    payload = cols // 2 if kind >= 2 else cols
    return payload + (4 if (kind & 1) else 8)


def fused_rowwise_quantize(data, kind):
    data = _c(data, np.float32)
    rows, cols = data.shape
    line = fused_line_bytes(cols, kind)
    out = np.zeros((rows, line), np.uint8)
    lib().orc_fused_rowwise_quantize(_ptr(data), _i64(rows), _i64(cols), C.c_int(kind), _ptr(out), _i64(line))
    return out


def _idx(indices):
    indices = np.ascontiguousarray(indices)
    if indices.dtype == np.int64:
        return indices, 1
    if indices.dtype == np.int32:
        return indices, 0
    raise TypeError("indices must be int32 or int64")


def frwq_slws_u8_f32(data, weights, indices, lengths, out_line=None):
    """CPU-backend kernel (UInt8FusedQTy, fp32): libjit.cpp:1253-1276."""
    data = _c(data, np.uint8)
    in_line = data.shape[1]
    out_line = in_line - 8 if out_line is None else out_line
    weights = _c(weights, np.float32)
    indices, idx64 = _idx(indices)
    lengths = _c(lengths, np.int32)
    dest = np.empty((lengths.shape[0], out_line), np.float32)
    lib().orc_frwq_slws_u8_f32(_ptr(dest), _ptr(data), _ptr(weights), _ptr(indices), C.c_int(idx64),
                               _ptr(lengths), _i64(lengths.shape[0]), _i64(in_line), _i64(out_line))
    return dest


def _out_cols(in_line, kind):
    payload = in_line - (4 if (kind & 1) else 8)
    return payload * 2 if kind >= 2 else payload


def frwq_slws_interp(data, kind, weights, indices, lengths, out_fp16=None, fp16_acc=False):
    """Interpreter kernel, every fused kind: InterpreterNodes.cpp:5764-5889.
    Result is float16 (numpy) when out_fp16 else float32; weights have the result's type."""
    data = _c(data, np.uint8)
    in_line = data.shape[1]
    out_line = _out_cols(in_line, kind)
    if out_fp16 is None:
        out_fp16 = bool(kind & 1)
    weights = _c(weights, np.float16 if out_fp16 else np.float32)
    indices, idx64 = _idx(indices)
    lengths = _c(lengths, np.int32)
    dest = np.empty((lengths.shape[0], out_line), np.float16 if out_fp16 else np.float32)
    lib().orc_frwq_slws_interp(_ptr(dest), _ptr(data), C.c_int(kind), _ptr(weights), _ptr(indices),
                               C.c_int(idx64), _ptr(lengths), _i64(lengths.shape[0]), _i64(in_line),
                               _i64(out_line), C.c_int(int(out_fp16)), C.c_int(int(fp16_acc)))
    return dest


def embedding_bag_byte_rowwise_offsets(data, kind, weights, indices, offsets, has_end_offset,
                                       out_fp16=None, fp16_acc=False, num_indices=None):
    data = _c(data, np.uint8)
    in_line = data.shape[1]
    out_line = _out_cols(in_line, kind)
    if out_fp16 is None:
        out_fp16 = bool(kind & 1)
    weights = _c(weights, np.float16 if out_fp16 else np.float32)
    indices, idx64 = _idx(indices)
    offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
    segs = offsets.shape[0]
    nseg_out = segs - 1 if has_end_offset else segs
    dest = np.zeros((nseg_out, out_line), np.float16 if out_fp16 else np.float32)
    n_idx = indices.shape[0] if num_indices is None else num_indices
    lib().orc_embedding_bag_byte_rowwise_offsets(
        _ptr(dest), _ptr(data), C.c_int(kind), _ptr(weights), _ptr(indices), _ptr(offsets), C.c_int(idx64),
        _i64(segs), _i64(n_idx), _i64(in_line), _i64(out_line), C.c_int(int(has_end_offset)),
        C.c_int(int(out_fp16)), C.c_int(int(fp16_acc)))
    return dest


def int_nbit_split_embedding_bags(dev_weights, uvm_weights, placements, weights_offsets, weights_tys,
                                  dim_offsets, total_dims, indices, offsets, pooling_mode=0,
                                  indice_weights=None, out_fp16=False, so_fp32=False, row_alignment=16):
    """Table-batched embedding bags (InterpreterNodes.cpp:6664-6738); result [B, total_dims]."""
    dev_weights, uvm_weights = _c(dev_weights, np.uint8), _c(uvm_weights, np.uint8)
    placements, dim_offsets = _c(placements, np.int32), _c(dim_offsets, np.int32)
    weights_tys = _c(weights_tys, np.uint8)
    weights_offsets, wo64 = _idx(weights_offsets)
    indices, idx64 = _idx(indices)
    offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
    T = dim_offsets.shape[0] - 1
    B = (offsets.shape[0] - 1) // T
    iw, iw16 = None, 0
    if indice_weights is not None:
        iw16 = int(np.asarray(indice_weights).dtype == np.float16)
        iw = _c(indice_weights, np.float16 if iw16 else np.float32)
    dest = np.empty((B, total_dims), np.float16 if out_fp16 else np.float32)
    lib().orc_int_nbit_split_embedding_bags(
        _ptr(dest), _ptr(dev_weights), _ptr(uvm_weights), _ptr(placements), _ptr(weights_offsets), C.c_int(wo64),
        _ptr(weights_tys), _ptr(dim_offsets), _i64(T), _i64(total_dims), _ptr(indices), _ptr(offsets),
        C.c_int(idx64), _i64(B), C.c_int(pooling_mode), _ptr(iw) if iw is not None else None, C.c_int(iw16),
        C.c_int(int(out_fp16)), C.c_int(int(so_fp32)), C.c_int(row_alignment))
    return dest


def dynamic_rowwise_quantized_fc(inp, weights_kn, bias, scales, offsets):
    """DynamicRowwiseQuantizedFullyConnected (InterpreterNodes.cpp:4677-4749): fp16 [M,K] x int8 [K,N]."""
    inp = _c(inp, np.float16)
    w = _c(weights_kn, np.int8)
    M, K = inp.shape
    N = w.shape[1]
    bias, scales, offsets = _c(bias, np.float32), _c(scales, np.float32), _c(offsets, np.int32)
    out = np.empty((M, N), np.float16)
    lib().orc_dynamic_rowwise_quantized_fc(_ptr(out), _ptr(inp), _ptr(w), _ptr(bias), _ptr(scales), _ptr(offsets),
                                           _i64(M), _i64(K), _i64(N))
    return out


def quantization_profile(x, comp_info, hist):
    """libjit_quantization_profile (libjit.cpp:3440-3523): returns the updated (comp_info, hist)."""
    x = _c(x, np.float32).reshape(-1)
    ci, h = _c(comp_info, np.float32).copy(), _c(hist, np.float32).copy()
    lib().orc_quantization_profile(_ptr(x), _i64(x.size), _ptr(ci), _ptr(h), _i64(h.size))
    return ci, h


def sparse_lengths_weighted_sum_f32(data, weights, indices, lengths):
    data = _c(data, np.float32)
    weights = _c(weights, np.float32)
    indices, idx64 = _idx(indices)
    lengths = _c(lengths, np.int32)
    dest = np.empty((lengths.shape[0], data.shape[1]), np.float32)
    lib().orc_sparse_lengths_weighted_sum_f32(_ptr(dest), _ptr(data), _ptr(weights), _ptr(indices),
                                              C.c_int(idx64), _ptr(lengths), _i64(lengths.shape[0]),
                                              _i64(data.shape[1]))
    return dest


def sparse_lengths_sum_f32(data, indices, lengths):
    data = _c(data, np.float32)
    indices, idx64 = _idx(indices)
    lengths = _c(lengths, np.int32)
    dest = np.empty((lengths.shape[0], data.shape[1]), np.float32)
    lib().orc_sparse_lengths_sum_f32(_ptr(dest), _ptr(data), _ptr(indices), C.c_int(idx64), _ptr(lengths),
                                     _i64(lengths.shape[0]), _i64(data.shape[1]))
    return dest


def rowwise_quantized_slws_f32(data, scales, offsets, weights, indices, lengths):
    data = _c(data, np.uint8)
    scales, offsets, weights = _c(scales, np.float32), _c(offsets, np.float32), _c(weights, np.float32)
    indices, idx64 = _idx(indices)
    lengths = _c(lengths, np.int32)
    dest = np.empty((lengths.shape[0], data.shape[1]), np.float32)
    lib().orc_rowwise_quantized_slws_f32(_ptr(dest), _ptr(data), _ptr(scales), _ptr(offsets), _ptr(weights),
                                         _ptr(indices), C.c_int(idx64), _ptr(lengths), _i64(lengths.shape[0]),
                                         _i64(data.shape[1]))
    return dest


# ---------------------------------------------------------------------------- dense int8
def _split_rows(M, threads):
    threads = max(1, min(threads, M))
    edges = np.linspace(0, M, threads + 1).astype(np.int64)
    return [(int(edges[t]), int(edges[t + 1])) for t in range(threads) if edges[t + 1] > edges[t]]


def _run_rows(M, threads, fn):
    parts = _split_rows(M, threads)
    if len(parts) == 1:
        fn(*parts[0])
        return
    with ThreadPoolExecutor(len(parts)) as ex:
        list(ex.map(lambda p: fn(*p), parts))


def rowwise_quantized_fc_i8_i32(inp, w, bias, w_offsets, bias_triples, out_triples, out_offset,
                                in_offset, bias_offset, threads=1):
    """libjit_matmul.cpp:284-316.  inp [M,K] int8, w [N,K] int8 -> [M,N] int8.
    The batch rows are split over `threads` host threads (ctypes drops the GIL)."""
    inp, w = _c(inp, np.int8), _c(w, np.int8)
    M, K = inp.shape
    N = w.shape[0]
    bias, w_offsets = _c(bias, np.int32), _c(w_offsets, np.int32)
    bt = [_c(a, np.int32) for a in bias_triples]
    ot = [_c(a, np.int32) for a in out_triples]
    out = np.empty((M, N), np.int8)
    f = lib().orc_rowwise_quantized_fc_i8_i32

    def run(lo, hi):
        f(_ptr(out[lo:hi]), _ptr(inp[lo:hi]), _ptr(w), _ptr(bias), _ptr(w_offsets), _ptr(bt[0]), _ptr(bt[1]),
          _ptr(bt[2]), _ptr(ot[0]), _ptr(ot[1]), _ptr(ot[2]), _i64(hi - lo), _i64(K), _i64(N),
          _i32(out_offset), _i32(in_offset), _i32(bias_offset))

    _run_rows(M, threads, run)
    return out


def fc_i8_i32(inp, w, bias, out_offset, in_offset, w_offset, bias_offset, bias_triple, out_triple, threads=1):
    """libjit_matmul.cpp:254-280.  inp [M,K], w [K,N]."""
    inp, w, bias = _c(inp, np.int8), _c(w, np.int8), _c(bias, np.int32)
    M, K = inp.shape
    N = w.shape[1]
    out = np.empty((M, N), np.int8)
    f = lib().orc_fc_i8_i32

    def run(lo, hi):
        f(_ptr(out[lo:hi]), _ptr(inp[lo:hi]), _ptr(w), _ptr(bias), _i64(hi - lo), _i64(K), _i64(N),
          _i32(out_offset), _i32(in_offset), _i32(w_offset), _i32(bias_offset),
          *[_i32(int(v)) for v in bias_triple], *[_i32(int(v)) for v in out_triple])

    _run_rows(M, threads, run)
    return out


def matmul_i8(lhs, rhs, out_offset, lhs_offset, rhs_offset, out_triple, threads=1):
    """libjit_matmul.cpp:353-371."""
    lhs, rhs = _c(lhs, np.int8), _c(rhs, np.int8)
    M, K = lhs.shape
    N = rhs.shape[1]
    out = np.empty((M, N), np.int8)
    f = lib().orc_matmul_i8

    def run(lo, hi):
        f(_ptr(out[lo:hi]), _ptr(lhs[lo:hi]), _ptr(rhs), _i64(hi - lo), _i64(K), _i64(N), _i32(out_offset),
          _i32(lhs_offset), _i32(rhs_offset), *[_i32(int(v)) for v in out_triple])

    _run_rows(M, threads, run)
    return out


def _dims(*v):
    return np.array(v, dtype=np.int64)


def conv2d_i8_i32(inp, filt, bias, out_hw, kernels, strides, pads, group, dilation, out_offset, in_offset,
                  filter_offsets, bias_offsets, bias_triples, out_triples, act_type=0, act_args=None,
                  per_channel=True):
    """libjit_conv.cpp:151-239 (per_channel) / :49-147.  inp NHWC int8, filt [outC,kH,kW,inC/g]."""
    inp, filt, bias = _c(inp, np.int8), _c(filt, np.int8), _c(bias, np.int32)
    n, ih, iw, ic = inp.shape
    oc = filt.shape[0]
    out = np.empty((n, out_hw[0], out_hw[1], oc), np.int8)
    fo, bo = _c(np.atleast_1d(filter_offsets), np.int32), _c(np.atleast_1d(bias_offsets), np.int32)
    bt = [_c(np.atleast_1d(a), np.int32) for a in bias_triples]
    ot = [_c(np.atleast_1d(a), np.int32) for a in out_triples]
    aa = _c(np.zeros(3) if act_args is None else act_args, np.int32)
    od, idm, fd = _dims(*out.shape), _dims(*inp.shape), _dims(*filt.shape)
    k, s, p, d = _dims(*kernels), _dims(*strides), _dims(*pads), _dims(*dilation)
    lib().orc_conv2d_i8_i32(_ptr(out), _ptr(inp), _ptr(filt), _ptr(bias), _ptr(od), _ptr(idm), _ptr(fd), _ptr(k),
                            _ptr(s), _ptr(p), _i64(group), _ptr(d), _i32(out_offset), _i32(in_offset),
                            C.c_int(int(per_channel)), _ptr(fo), _ptr(bo), _ptr(bt[0]), _ptr(bt[1]), _ptr(bt[2]),
                            _ptr(ot[0]), _ptr(ot[1]), _ptr(ot[2]), _i32(act_type), _ptr(aa))
    return out


# ---------------------------------------------------------------------------- int8 glue
def element_add_i8(lhs, rhs, dest_offset, lhs_offset, rhs_offset, lhs_triple, rhs_triple):
    lhs, rhs = _c(lhs, np.int8), _c(rhs, np.int8)
    out = np.empty_like(lhs)
    lib().orc_element_add_i8(_ptr(out), _ptr(lhs), _ptr(rhs), _i64(lhs.size), _i32(dest_offset), _i32(lhs_offset),
                             _i32(rhs_offset), *[_i32(int(v)) for v in lhs_triple],
                             *[_i32(int(v)) for v in rhs_triple])
    return out


def element_binary_i8(op, lhs, rhs, dest_offset, lhs_offset, rhs_offset, lhs_triple, rhs_triple):
    """op 0 add, 1 sub, 2 max, 3 min."""
    lhs, rhs = _c(lhs, np.int8), _c(rhs, np.int8)
    out = np.empty_like(lhs)
    lib().orc_element_binary_i8(C.c_int(op), _ptr(out), _ptr(lhs), _ptr(rhs), _i64(lhs.size), _i32(dest_offset),
                                _i32(lhs_offset), _i32(rhs_offset), *[_i32(int(v)) for v in lhs_triple],
                                *[_i32(int(v)) for v in rhs_triple])
    return out


def element_muldiv_i8(is_div, lhs, rhs, dest_offset, lhs_offset, rhs_offset, triple):
    lhs, rhs = _c(lhs, np.int8), _c(rhs, np.int8)
    out = np.empty_like(lhs)
    lib().orc_element_muldiv_i8(C.c_int(int(is_div)), _ptr(out), _ptr(lhs), _ptr(rhs), _i64(lhs.size), _i32(dest_offset),
                                _i32(lhs_offset), _i32(rhs_offset), *[_i32(int(v)) for v in triple])
    return out


def batched_add_i8(batch, slice_, dest_offset, batch_offset, slice_offset, batch_triple, slice_triple):
    batch = _c(batch, np.int8)
    is32 = np.asarray(slice_).dtype == np.int32
    slice_ = _c(slice_, np.int32 if is32 else np.int8)
    out = np.empty_like(batch)
    lib().orc_batched_add_i8(_ptr(out), _ptr(batch), _ptr(slice_), C.c_int(int(is32)), _i64(batch.shape[0]),
                             _i64(batch.size // max(batch.shape[0], 1)), _i32(dest_offset), _i32(batch_offset),
                             _i32(slice_offset), *[_i32(int(v)) for v in batch_triple],
                             *[_i32(int(v)) for v in slice_triple])
    return out


def element_relu_i8(src, src_offset, dest_offset, triple):
    src = _c(src, np.int8)
    out = np.empty_like(src)
    lib().orc_element_relu_i8(_ptr(out), _ptr(src), _i64(src.size), _i32(src_offset), _i32(dest_offset),
                              *[_i32(int(v)) for v in triple])
    return out


def element_maxsplat_i8(src, splat):
    src = _c(src, np.int8)
    out = np.empty_like(src)
    lib().orc_element_maxsplat_i8(_ptr(out), _ptr(src), _i64(src.size), C.c_int8(int(splat)))
    return out


def element_rescale_i8(src, out_offset, in_offset, triple):
    src = _c(src, np.int8)
    out = np.empty_like(src)
    lib().orc_element_rescale_i8(_ptr(out), _ptr(src), _i64(src.size), _i32(out_offset), _i32(in_offset),
                                 *[_i32(int(v)) for v in triple])
    return out


def element_quantize_i8(src, scale, offset):
    src = _c(src, np.float32)
    out = np.empty(src.shape, np.int8)
    lib().orc_element_quantize_i8(_ptr(out), _ptr(src), _i64(src.size), _f32(scale), _i32(offset))
    return out


def element_dequantize_i8(src, scale, offset):
    src = _c(src, np.int8)
    out = np.empty(src.shape, np.float32)
    lib().orc_element_dequantize_i8(_ptr(out), _ptr(src), _i64(src.size), _f32(scale), _i32(offset))
    return out


def max_pool_i8(inp, out_hw, kernels, strides, pads, out_offset):
    inp = _c(inp, np.int8)
    out = np.empty((inp.shape[0], out_hw[0], out_hw[1], inp.shape[3]), np.int8)
    lib().orc_max_pool_i8(_ptr(inp), _ptr(out), _ptr(_dims(*inp.shape)), _ptr(_dims(*out.shape)),
                          _ptr(_dims(*kernels)), _ptr(_dims(*strides)), _ptr(_dims(*pads)), _i32(out_offset))
    return out


def avg_pool_i8(inp, out_hw, kernels, strides, pads, count_include_pads, out_offset, in_offset, triple):
    inp = _c(inp, np.int8)
    out = np.empty((inp.shape[0], out_hw[0], out_hw[1], inp.shape[3]), np.int8)
    lib().orc_avg_pool_i8(_ptr(inp), _ptr(out), _ptr(_dims(*inp.shape)), _ptr(_dims(*out.shape)),
                          _ptr(_dims(*kernels)), _ptr(_dims(*strides)), _ptr(_dims(*pads)),
                          C.c_int(int(count_include_pads)), _i32(out_offset), _i32(in_offset),
                          *[_i32(int(v)) for v in triple])
    return out


def pairwise_dot_interaction(dense, pooled):
    dense, pooled = _c(dense, np.float32), _c(pooled, np.float32)
    B, D = dense.shape
    T = pooled.size // (B * D)
    n = T + 1
    out = np.empty((B, D + n * (n - 1) // 2), np.float32)
    lib().orc_pairwise_dot_interaction(_ptr(dense), _ptr(pooled), _i64(B), _i64(T), _i64(D), _ptr(out))
    return out


# ---------------------------------------------------------------------------- reference libjit
class LibjitRef:
    """Calls into the reference's own libjit build (dim_t = uint64)."""

    def __init__(self, flavour="strict"):
        self.l = ref(flavour)
        if self.l is None:
            raise RuntimeError("oracle/_ref/libjit_%s.so is not built" % flavour)

    @staticmethod
    def _d(*v):
        return np.array(v, dtype=np.uint64)

    def frwq_slws(self, data, weights, indices, lengths):
        data = _c(data, np.uint8)
        in_line = data.shape[1]
        out_line = in_line - 8
        weights = _c(weights, np.float32)
        indices, idx64 = _idx(indices)
        lengths = _c(lengths, np.int32)
        dest = np.empty((lengths.shape[0], out_line), np.float32)
        fn = (self.l.libjit_fused_rowwise_quantized_sparse_lengths_weighted_sum_f_u if idx64
              else self.l.libjit_fused_rowwise_quantized_sparse_lengths_weighted_sum_f_i32)
        fn(_ptr(dest), _ptr(data), _ptr(weights), _ptr(indices), _ptr(lengths), C.c_uint64(lengths.shape[0]),
           C.c_uint64(in_line), C.c_uint64(out_line))
        return dest

    def sparse_lengths_weighted_sum(self, data, weights, indices, lengths):
        """libjit_sparse_lengths_weighted_sum_f_u / _f_i32; weights None -> libjit_sparse_lengths_sum_*."""
        data = _c(data, np.float32)
        indices, idx64 = _idx(indices)
        lengths = _c(lengths, np.int32)
        dest = np.empty((lengths.shape[0], data.shape[1]), np.float32)
        sfx = "f_u" if idx64 else "f_i32"
        if weights is None:
            getattr(self.l, "libjit_sparse_lengths_sum_" + sfx)(
                _ptr(dest), _ptr(data), _ptr(indices), _ptr(lengths), C.c_uint64(lengths.shape[0]),
                C.c_uint64(data.shape[1]))
        else:
            weights = _c(weights, np.float32)
            getattr(self.l, "libjit_sparse_lengths_weighted_sum_" + sfx)(
                _ptr(dest), _ptr(data), _ptr(weights), _ptr(indices), _ptr(lengths), C.c_uint64(lengths.shape[0]),
                C.c_uint64(data.shape[1]))
        return dest

    def rowwise_quantized_slws(self, data, scales, offsets, weights, indices, lengths):
        data = _c(data, np.uint8)
        scales, offsets, weights = _c(scales, np.float32), _c(offsets, np.float32), _c(weights, np.float32)
        indices, idx64 = _idx(indices)
        lengths = _c(lengths, np.int32)
        dest = np.empty((lengths.shape[0], data.shape[1]), np.float32)
        fn = getattr(self.l, "libjit_rowwise_quantized_sparse_lengths_weighted_sum_" + ("f_u" if idx64 else "f_i32"))
        fn(_ptr(dest), _ptr(data), _ptr(scales), _ptr(offsets), _ptr(weights), _ptr(indices), _ptr(lengths),
           C.c_uint64(lengths.shape[0]), C.c_uint64(data.shape[1]))
        return dest

    def quantization_profile(self, x, comp_info, hist):
        x = _c(x, np.float32).reshape(-1)
        ci, h = _c(comp_info, np.float32).copy(), _c(hist, np.float32).copy()
        dims = (C.c_uint64 * 1)(h.size)
        self.l.libjit_quantization_profile(_ptr(x), C.c_uint64(x.size), _ptr(ci), _ptr(h), dims)
        return ci, h

    def embedding_bag_byte_rowwise_offsets(self, data, weights, indices, offsets, has_end_offset):
        data = _c(data, np.uint8)
        in_line = data.shape[1]
        out_line = in_line - 8
        weights = _c(weights, np.float32)
        indices, offsets = _c(indices, np.int32), _c(offsets, np.int32)
        segs = offsets.shape[0]
        dest = np.zeros((segs - 1 if has_end_offset else segs, out_line), np.float32)
        self.l.libjit_embedding_bag_byte_rowwise_offsets_f(
            _ptr(dest), _ptr(data), _ptr(weights), _ptr(indices), _ptr(offsets), C.c_uint64(segs),
            C.c_uint64(indices.shape[0]), C.c_uint64(in_line), C.c_uint64(out_line), C.c_bool(bool(has_end_offset)))
        return dest

    def rowwise_quantized_fc_i8_i32(self, inp, w, bias, w_offsets, bias_triples, out_triples, out_offset,
                                    in_offset, bias_offset, threads=1):
        inp, w = _c(inp, np.int8), _c(w, np.int8)
        M, K = inp.shape
        N = w.shape[0]
        bias, w_offsets = _c(bias, np.int32), _c(w_offsets, np.int32)
        bt = [_c(a, np.int32) for a in bias_triples]
        ot = [_c(a, np.int32) for a in out_triples]
        out = np.empty((M, N), np.int8)
        wd, bd = self._d(N, K), self._d(N)

        def run(lo, hi):
            od, idm = self._d(hi - lo, N), self._d(hi - lo, K)
            self.l.libjit_rowwise_quantized_fc_i8_i32(
                _ptr(out[lo:hi]), _ptr(inp[lo:hi]), _ptr(w), _ptr(bias), _ptr(w_offsets), _ptr(bt[0]), _ptr(bt[1]),
                _ptr(bt[2]), _ptr(ot[0]), _ptr(ot[1]), _ptr(ot[2]), _ptr(od), _ptr(idm), _ptr(wd), _ptr(bd),
                C.c_uint64(N), _i32(out_offset), _i32(in_offset), _i32(bias_offset))

        _run_rows(M, threads, run)
        return out

    def fc_i8_i32(self, inp, w, bias, out_offset, in_offset, w_offset, bias_offset, bias_triple, out_triple):
        inp, w, bias = _c(inp, np.int8), _c(w, np.int8), _c(bias, np.int32)
        M, K = inp.shape
        N = w.shape[1]
        out = np.empty((M, N), np.int8)
        self.l.libjit_fc_i8_i32(_ptr(out), _ptr(inp), _ptr(w), _ptr(bias), _ptr(self._d(M, N)), _ptr(self._d(M, K)),
                                _ptr(self._d(K, N)), _ptr(self._d(N)), _i32(out_offset), _i32(in_offset),
                                _i32(w_offset), _i32(bias_offset), *[_i32(int(v)) for v in bias_triple],
                                *[_i32(int(v)) for v in out_triple])
        return out

    def matmul_i8(self, lhs, rhs, out_offset, lhs_offset, rhs_offset, out_triple):
        lhs, rhs = _c(lhs, np.int8), _c(rhs, np.int8)
        M, K = lhs.shape
        N = rhs.shape[1]
        out = np.empty((M, N), np.int8)
        self.l.libjit_matmul_i8(_ptr(out), _ptr(lhs), _ptr(rhs), _ptr(self._d(M, N)), _ptr(self._d(M, K)),
                                _ptr(self._d(K, N)), _i32(out_offset), _i32(lhs_offset), _i32(rhs_offset),
                                *[_i32(int(v)) for v in out_triple])
        return out

    def channelwise_quantized_conv2d_i8_i32(self, inp, filt, bias, out_hw, kernels, strides, pads, group, dilation,
                                            out_offset, in_offset, filter_offsets, bias_offsets, bias_triples,
                                            out_triples, act_type=0, act_args=None):
        inp, filt, bias = _c(inp, np.int8), _c(filt, np.int8), _c(bias, np.int32)
        oc = filt.shape[0]
        out = np.empty((inp.shape[0], out_hw[0], out_hw[1], oc), np.int8)
        fo, bo = _c(filter_offsets, np.int32), _c(bias_offsets, np.int32)
        bt = [_c(a, np.int32) for a in bias_triples]
        ot = [_c(a, np.int32) for a in out_triples]
        aa = _c(np.zeros(3) if act_args is None else act_args, np.int32)
        self.l.libjit_channelwise_quantized_conv2d_i8_i32(
            _ptr(out), _ptr(inp), _ptr(filt), _ptr(bias), _ptr(self._d(*out.shape)), _ptr(self._d(*inp.shape)),
            _ptr(self._d(*filt.shape)), _ptr(self._d(oc)), _ptr(self._d(*kernels)), _ptr(self._d(*strides)),
            _ptr(self._d(*pads)), C.c_uint64(group), _ptr(self._d(*dilation)), _i32(out_offset), _i32(in_offset),
            _ptr(fo), _ptr(bo), _ptr(bt[0]), _ptr(bt[1]), _ptr(bt[2]), _ptr(ot[0]), _ptr(ot[1]), _ptr(ot[2]),
            _i32(act_type), _ptr(aa))
        return out

    def conv2d_i8_i32(self, inp, filt, bias, out_hw, kernels, strides, pads, group, dilation, out_offset, in_offset,
                      filter_offset, bias_offset, bias_triple, out_triple, act_type=0, act_args=None,
                      depth_unroll=1):
        inp, filt, bias = _c(inp, np.int8), _c(filt, np.int8), _c(bias, np.int32)
        oc = filt.shape[0]
        out = np.empty((inp.shape[0], out_hw[0], out_hw[1], oc), np.int8)
        aa = _c(np.zeros(3) if act_args is None else act_args, np.int32)
        self.l.libjit_conv2d_i8_i32(
            _ptr(out), _ptr(inp), _ptr(filt), _ptr(bias), _ptr(self._d(*out.shape)), _ptr(self._d(*inp.shape)),
            _ptr(self._d(*filt.shape)), _ptr(self._d(oc)), _ptr(self._d(*kernels)), _ptr(self._d(*strides)),
            _ptr(self._d(*pads)), C.c_uint64(group), _i32(out_offset), _i32(in_offset), _i32(filter_offset),
            _i32(bias_offset), *[_i32(int(v)) for v in bias_triple], *[_i32(int(v)) for v in out_triple],
            C.c_uint(depth_unroll), _ptr(self._d(*dilation)), _i32(act_type), _ptr(aa))
        return out

    def max_pool_i8(self, inp, out_hw, kernels, strides, pads, out_offset):
        inp = _c(inp, np.int8)
        out = np.empty((inp.shape[0], out_hw[0], out_hw[1], inp.shape[3]), np.int8)
        self.l.libjit_max_pool_i8(_ptr(inp), _ptr(out), _ptr(self._d(*inp.shape)), _ptr(self._d(*out.shape)),
                                  _ptr(self._d(*kernels)), _ptr(self._d(*strides)), _ptr(self._d(*pads)),
                                  _i32(out_offset))
        return out

    def avg_pool_i8(self, inp, out_hw, kernels, strides, pads, count_include_pads, out_offset, in_offset, triple):
        inp = _c(inp, np.int8)
        out = np.empty((inp.shape[0], out_hw[0], out_hw[1], inp.shape[3]), np.int8)
        self.l.libjit_avg_pool_i8(_ptr(inp), _ptr(out), _ptr(self._d(*inp.shape)), _ptr(self._d(*out.shape)),
                                  _ptr(self._d(*kernels)), _ptr(self._d(*strides)), _ptr(self._d(*pads)),
                                  C.c_bool(bool(count_include_pads)), _i32(out_offset), _i32(in_offset),
                                  *[_i32(int(v)) for v in triple])
        return out

    def _elem(self, name, restype, n, *args):
        fn = getattr(self.l, name)
        fn.restype = restype
        return [fn(C.c_uint64(i), *args) for i in range(n)]

    def element_add_i8(self, lhs, rhs, dest_offset, lhs_offset, rhs_offset, lhs_triple, rhs_triple):
        lhs, rhs = _c(lhs, np.int8), _c(rhs, np.int8)
        r = self._elem("libjit_element_add_kernel_i8", C.c_int8, lhs.size, _ptr(lhs), _ptr(rhs), _i32(dest_offset),
                       _i32(lhs_offset), _i32(rhs_offset), *[_i32(int(v)) for v in lhs_triple],
                       *[_i32(int(v)) for v in rhs_triple])
        return np.array(r, np.int8).reshape(lhs.shape)

    def element_binary_i8(self, op, lhs, rhs, dest_offset, lhs_offset, rhs_offset, lhs_triple, rhs_triple):
        lhs, rhs = _c(lhs, np.int8), _c(rhs, np.int8)
        name = "libjit_element_%s_kernel_i8" % ("add", "sub", "max", "min")[op]
        r = self._elem(name, C.c_int8, lhs.size, _ptr(lhs), _ptr(rhs), _i32(dest_offset), _i32(lhs_offset),
                       _i32(rhs_offset), *[_i32(int(v)) for v in lhs_triple], *[_i32(int(v)) for v in rhs_triple])
        return np.array(r, np.int8).reshape(lhs.shape)

    def element_muldiv_i8(self, is_div, lhs, rhs, dest_offset, lhs_offset, rhs_offset, triple):
        lhs, rhs = _c(lhs, np.int8), _c(rhs, np.int8)
        name = "libjit_element_%s_kernel_i8" % ("div" if is_div else "mul")
        r = self._elem(name, C.c_int8, lhs.size, _ptr(lhs), _ptr(rhs), _i32(dest_offset), _i32(lhs_offset),
                       _i32(rhs_offset), *[_i32(int(v)) for v in triple])
        return np.array(r, np.int8).reshape(lhs.shape)

    def batched_add_i8(self, batch, slice_, dest_offset, batch_offset, slice_offset, batch_triple, slice_triple):
        batch = _c(batch, np.int8)
        is32 = np.asarray(slice_).dtype == np.int32
        slice_ = _c(slice_, np.int32 if is32 else np.int8)
        out = np.empty_like(batch)
        fn = self.l.libjit_batchedadd_i32_i8 if is32 else self.l.libjit_batchedadd_i8
        fn(_ptr(out), _ptr(batch), _ptr(slice_), C.c_uint64(batch.shape[0]), C.c_uint64(batch.size // batch.shape[0]),
           _i32(dest_offset), _i32(batch_offset), _i32(slice_offset), *[_i32(int(v)) for v in batch_triple],
           *[_i32(int(v)) for v in slice_triple])
        return out

    def element_quantize_i8(self, src, scale, offset):
        src = _c(src, np.float32)
        r = self._elem("libjit_element_quantize_kernel_i8", C.c_int8, src.size, _ptr(src), _f32(scale), _i32(offset))
        return np.array(r, np.int8).reshape(src.shape)

    def element_rescale_i8(self, src, out_offset, in_offset, triple):
        src = _c(src, np.int8)
        r = self._elem("libjit_element_rescale_kernel_i8", C.c_int8, src.size, _ptr(src), _i32(out_offset),
                       _i32(in_offset), *[_i32(int(v)) for v in triple])
        return np.array(r, np.int8).reshape(src.shape)

    def element_relu_i8(self, src, src_offset, dest_offset, triple):
        src = _c(src, np.int8)
        r = self._elem("libjit_element_relu_i8", C.c_int8, src.size, _ptr(src), C.c_int8(src_offset),
                       C.c_int8(dest_offset), *[_i32(int(v)) for v in triple])
        return np.array(r, np.int8).reshape(src.shape)
