"""ctypes front end of the host runtime (glowb200_function_* / glowb200_device_manager_*).

`Function` builds what Backend::compile would hand to a device manager -- symbols and a flat
instruction list -- and `DeviceManager` is the addNetwork / evictNetwork / runFunction object.
The helper methods only marshal arguments; parameter derivation and execution are in the
library (glow_b200/csrc/runtime.cu).
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import GlowB200Error

CONSTANT, PLACEHOLDER, ACTIVATION, STATIC = 0, 1, 2, 3
(FRWQ_SLWS, RWQ_FC, CWQ_CONV, ADD, MAXSPLAT, QUANTIZE, DEQUANTIZE, MAXPOOL, AVGPOOL, TRANSPOSE, COPY) = range(1, 12)
(ADD_MAXSPLAT, RELU, RESCALE, FC_I8, MATMUL_I8, SPLAT, INSERT_TENSOR, PAIRWISE_DOT, SLWS_F32, RWQ_SLWS,
 EMBEDDING_BAG, SPLIT_EMBEDDING, DYN_QUANTIZED_FC, BINARY_I8, MULDIV_I8, BATCHED_ADD_I8) = range(12, 28)

RUNTIME_ERROR, OUT_OF_DEVICE_MEMORY, NET_NOT_FOUND, DEVICE_NONRECOVERABLE = 101, 102, 103, 104


def _check(rc):
    if rc != 0:
        raise GlowB200Error(rc, _lib.lib().glowb200_last_error().decode())


class Function:
    def __init__(self, name):
        self.name = name
        self.h = _lib.lib().glowb200_function_create(name.encode())
        self.sizes = {}

    def __del__(self):
        if getattr(self, "h", None):
            _lib.lib().glowb200_function_destroy(self.h)
            self.h = None

    def _symbol(self, name, kind, nbytes, data=None):
        sid = _lib.lib().glowb200_function_add_symbol(self.h, name.encode(), kind, int(nbytes),
                                                      None if data is None else C.c_void_p(data.ctypes.data))
        if sid < 0:
            raise GlowB200Error(RUNTIME_ERROR, _lib.lib().glowb200_last_error().decode())
        self.sizes[name] = int(nbytes)
        return sid

    def constant(self, name, array):
        a = np.ascontiguousarray(array)
        return self._symbol(name, CONSTANT, a.nbytes, a)

    def placeholder(self, name, nbytes):
        return self._symbol(name, PLACEHOLDER, nbytes)

    def activation(self, name, nbytes):
        return self._symbol(name, ACTIVATION, nbytes)

    def static_placeholder(self, name, nbytes):
        """A placeholder written once (transfer_static_placeholder) and shared by all contexts."""
        return self._symbol(name, STATIC, nbytes)

    def instruction(self, kind, operands, int_attrs=(), float_attrs=()):
        """operands: symbol ids, or (symbol id, byte offset) pairs for views of a larger tensor."""
        ids = [o[0] if isinstance(o, tuple) else o for o in operands]
        offs = [int(o[1]) if isinstance(o, tuple) else 0 for o in operands]
        ops = (C.c_int32 * len(ids))(*ids)
        of = (C.c_int64 * max(1, len(offs)))(*offs)
        ia = (C.c_int64 * max(1, len(int_attrs)))(*[int(v) for v in int_attrs])
        fa = (C.c_float * max(1, len(float_attrs)))(*[float(v) for v in float_attrs])
        if any(offs):
            _check(_lib.lib().glowb200_function_add_instruction_views(self.h, kind, ops, of, len(ids), ia, len(int_attrs),
                                                                      fa, len(float_attrs)))
        else:
            _check(_lib.lib().glowb200_function_add_instruction(self.h, kind, ops, len(ids), ia, len(int_attrs), fa,
                                                                len(float_attrs)))

    # readable wrappers over the attribute layouts documented in runtime.cu
    def frwq_slws(self, dest, data, weights, indices, lengths, *, kind, rows, in_line, out_line, segments, num_indices,
                  idx64=True, out_fp16=False, fp16_acc=False):
        self.instruction(FRWQ_SLWS, [dest, data, weights, indices, lengths],
                         [kind, rows, in_line, out_line, segments, num_indices, int(idx64), int(out_fp16), int(fp16_acc)])

    def rowwise_fc(self, dest, src, weights, scales, offsets, bias, *, M, K, N, in_tqp, bias_tqp, out_tqp, relu=False):
        self.instruction(RWQ_FC, [dest, src, weights, scales, offsets, bias],
                         [M, K, N, in_tqp[1], bias_tqp[1], out_tqp[1], int(relu)], [in_tqp[0], bias_tqp[0], out_tqp[0]])

    def channelwise_conv(self, dest, src, filt, bias, filter_scales, filter_offsets, bias_scales, bias_offsets, *, in_dims,
                         out_dims, kernels, strides, pads, group=1, dilation=(1, 1), in_tqp, out_tqp, act=0):
        n, h, w, c = in_dims
        _, oh, ow, oc = out_dims
        self.instruction(CWQ_CONV, [dest, src, filt, bias, filter_scales, filter_offsets, bias_scales, bias_offsets],
                         [n, h, w, c, oh, ow, oc, kernels[0], kernels[1], strides[0], strides[1], pads[0], pads[1], pads[2],
                          pads[3], group, dilation[0], dilation[1], in_tqp[1], out_tqp[1], act], [in_tqp[0], out_tqp[0]])

    def add(self, dest, lhs, rhs, *, n, lhs_tqp, rhs_tqp, dest_tqp):
        self.instruction(ADD, [dest, lhs, rhs], [n, dest_tqp[1], lhs_tqp[1], rhs_tqp[1]], [lhs_tqp[0], rhs_tqp[0], dest_tqp[0]])

    def maxsplat(self, dest, src, *, n, splat):
        self.instruction(MAXSPLAT, [dest, src], [n, splat])

    def quantize(self, dest, src, *, n, tqp):
        self.instruction(QUANTIZE, [dest, src], [n, tqp[1]], [tqp[0]])

    def dequantize(self, dest, src, *, n, tqp):
        self.instruction(DEQUANTIZE, [dest, src], [n, tqp[1]], [tqp[0]])

    def maxpool(self, dest, src, *, in_dims, out_hw, kernels, strides, pads, out_offset):
        n, h, w, c = in_dims
        self.instruction(MAXPOOL, [dest, src], [n, h, w, c, out_hw[0], out_hw[1], kernels[0], kernels[1], strides[0], strides[1],
                                                pads[0], pads[1], out_offset])

    def avgpool(self, dest, src, *, in_dims, out_hw, kernels, strides, pads, in_tqp, out_tqp, count_include_pads=True):
        n, h, w, c = in_dims
        self.instruction(AVGPOOL, [dest, src], [n, h, w, c, out_hw[0], out_hw[1], kernels[0], kernels[1], strides[0], strides[1],
                                                pads[0], pads[1], in_tqp[1], out_tqp[1], int(count_include_pads)],
                         [in_tqp[0], out_tqp[0]])

    def transpose(self, dest, src, *, dims, shuffle, elem_bytes):
        d = list(dims) + [1] * (4 - len(dims))
        s = list(shuffle) + [0] * (4 - len(shuffle))
        self.instruction(TRANSPOSE, [dest, src], [len(dims), elem_bytes] + d + s)

    def copy(self, dest, src, *, nbytes):
        self.instruction(COPY, [dest, src], [nbytes])

    def add_maxsplat(self, dest, lhs, rhs, *, n, lhs_tqp, rhs_tqp, dest_tqp, splat):
        self.instruction(ADD_MAXSPLAT, [dest, lhs, rhs], [n, dest_tqp[1], lhs_tqp[1], rhs_tqp[1], splat],
                         [lhs_tqp[0], rhs_tqp[0], dest_tqp[0]])

    def relu(self, dest, src, *, n, src_tqp, dest_tqp):
        self.instruction(RELU, [dest, src], [n, src_tqp[1], dest_tqp[1]], [src_tqp[0], dest_tqp[0]])

    def rescale(self, dest, src, *, n, in_tqp, out_tqp):
        self.instruction(RESCALE, [dest, src], [n, in_tqp[1], out_tqp[1]], [in_tqp[0], out_tqp[0]])

    def fully_connected(self, dest, src, weights, bias, *, M, K, N, in_tqp, w_tqp, bias_tqp, out_tqp):
        """weights: int8 [K, N] (Glow's FullyConnected layout)."""
        self.instruction(FC_I8, [dest, src, weights, bias], [M, K, N, in_tqp[1], w_tqp[1], bias_tqp[1], out_tqp[1]],
                         [in_tqp[0], w_tqp[0], bias_tqp[0], out_tqp[0]])

    def matmul(self, dest, lhs, rhs, *, M, K, N, lhs_tqp, rhs_tqp, out_tqp):
        self.instruction(MATMUL_I8, [dest, lhs, rhs], [M, K, N, lhs_tqp[1], rhs_tqp[1], out_tqp[1]],
                         [lhs_tqp[0], rhs_tqp[0], out_tqp[0]])

    def splat(self, dest, *, n, value, fp16=False):
        self.instruction(SPLAT, [dest], [n, int(fp16)], [value])

    def insert_tensor(self, dest, src, *, rows, width_bytes, dest_pitch_bytes, dest_offset_bytes):
        self.instruction(INSERT_TENSOR, [dest, src], [rows, width_bytes, dest_pitch_bytes, dest_offset_bytes])

    def pairwise_dot(self, dest, dense, pooled, *, batch, tables, dim, ld_out=None, quant=None):
        width = dim + (tables + 1) * tables // 2
        self.instruction(PAIRWISE_DOT, [dest, dense, pooled],
                         [batch, tables, dim, dim, tables * dim, width if ld_out is None else ld_out, int(quant is not None),
                          quant[1] if quant else 0], [quant[0] if quant else 1.0])

    def sparse_lengths_sum(self, dest, data, weights, indices, lengths, *, rows, line, segments, num_indices, idx64=True):
        """weights None: SparseLengthsSum."""
        self.instruction(SLWS_F32, [dest, data, -1 if weights is None else weights, indices, lengths],
                         [rows, line, segments, num_indices, int(idx64)])

    def rowwise_quantized_slws(self, dest, data, scales, offsets, weights, indices, lengths, *, rows, line, segments,
                               num_indices, idx64=True):
        self.instruction(RWQ_SLWS, [dest, data, scales, offsets, weights, indices, lengths],
                         [rows, line, segments, num_indices, int(idx64)])

    def embedding_bag(self, dest, data, weights, indices, offsets, *, kind, rows, in_line, out_line, num_offsets, num_indices,
                      idx64=True, has_end_offset=True, out_fp16=False, fp16_acc=False):
        self.instruction(EMBEDDING_BAG, [dest, data, weights, indices, offsets],
                         [kind, rows, in_line, out_line, num_offsets, num_indices, int(idx64), int(has_end_offset),
                          int(out_fp16), int(fp16_acc)])

    def split_embedding_bags(self, dest, dev_weights, uvm_weights, placements, weights_offsets, weights_tys, dim_offsets,
                             indices, offsets, indice_weights=None, *, dev_bytes, uvm_bytes, num_tables, total_dims,
                             num_indices, bags_per_table, idx64=False, weights_offsets_are_int64=False, pooling_mode=0,
                             indice_weights_are_fp16=False, out_fp16=False, scale_offset_is_fp32=False, row_alignment=16):
        """IntNBitSplitEmbeddingBags; with indice_weights: IntNBitSplitEmbeddingWeightedBags."""
        self.instruction(SPLIT_EMBEDDING,
                         [dest, dev_weights, uvm_weights, placements, weights_offsets, weights_tys, dim_offsets, indices,
                          offsets, -1 if indice_weights is None else indice_weights],
                         [dev_bytes, uvm_bytes, num_tables, total_dims, num_indices, bags_per_table, int(idx64),
                          int(weights_offsets_are_int64), pooling_mode, int(indice_weights_are_fp16), int(out_fp16),
                          int(scale_offset_is_fp32), row_alignment])

    def dynamic_quantized_fc(self, dest, src, weights, bias, scales=None, offsets=None, *, M, K, N, weights_tqp=(0.0, 0)):
        """DynamicRowwiseQuantizedFullyConnected (scales / offsets per output column) or, without them,
        DynamicQuantizedFullyConnected (weights_tqp = the weights' scale and offset).  weights: int8 [K, N]."""
        self.instruction(DYN_QUANTIZED_FC, [dest, src, weights, bias, -1 if scales is None else scales,
                                            -1 if offsets is None else offsets], [M, K, N, weights_tqp[1]], [weights_tqp[0]])

    def binary(self, op, dest, lhs, rhs, *, n, lhs_tqp, rhs_tqp, dest_tqp):
        """ElementAdd / Sub / Max / Min (op: ops.BINARY_*) on int8 tensors."""
        self.instruction(BINARY_I8, [dest, lhs, rhs], [n, dest_tqp[1], lhs_tqp[1], rhs_tqp[1], op],
                         [lhs_tqp[0], rhs_tqp[0], dest_tqp[0]])

    def muldiv(self, is_div, dest, lhs, rhs, *, n, lhs_tqp, rhs_tqp, dest_tqp):
        self.instruction(MULDIV_I8, [dest, lhs, rhs], [n, dest_tqp[1], lhs_tqp[1], rhs_tqp[1], int(bool(is_div))],
                         [lhs_tqp[0], rhs_tqp[0], dest_tqp[0]])

    def batched_add(self, dest, batch, slice_, *, num_slices, slice_size, batch_tqp, slice_tqp, dest_tqp, slice_is_int32=False):
        self.instruction(BATCHED_ADD_I8, [dest, batch, slice_],
                         [num_slices, slice_size, dest_tqp[1], batch_tqp[1], slice_tqp[1], int(slice_is_int32)],
                         [batch_tqp[0], slice_tqp[0], dest_tqp[0]])

    def compile(self):
        _check(_lib.lib().glowb200_function_compile(self.h))
        return self

    @property
    def batched_pooling_launches(self):
        return int(_lib.lib().glowb200_function_batched_pooling_launches(self.h))

    @property
    def fused_quantize_transposes(self):
        return int(_lib.lib().glowb200_function_fused_quantize_transposes(self.h))

    @property
    def constant_bytes(self):
        return int(_lib.lib().glowb200_function_constant_bytes(self.h))


class DeviceManager:
    def __init__(self, device_id=0, max_memory_bytes=0):
        self.h = _lib.lib().glowb200_device_manager_create(int(device_id), int(max_memory_bytes))
        self._functions = {}
        self._io = []
        self._inflight = {}

    def init(self):
        _check(_lib.lib().glowb200_device_manager_init(self.h))
        return self

    def add_network(self, fn):
        _check(_lib.lib().glowb200_device_manager_add_network(self.h, fn.h))
        self._functions[fn.name] = fn  # the device manager borrows the function

    def evict_network(self, name):
        _check(_lib.lib().glowb200_device_manager_evict_network(self.h, name.encode()))
        self._functions.pop(name, None)

    def run_function(self, name, bindings, outputs=None):
        """bindings: dict placeholder name -> numpy array.  outputs=None: every array is copied in
        and written back; else the names in `outputs` are copied out only, the others in only."""
        names = list(bindings)
        arrs = [bindings[k] for k in names]
        for a in arrs:
            if not (isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"] and a.flags["WRITEABLE"]):
                raise TypeError("bindings must be writable C-contiguous numpy arrays")
        cn = (C.c_char_p * len(names))(*[k.encode() for k in names])
        cb = (C.c_void_p * len(names))(*[a.ctypes.data for a in arrs])
        cs = (C.c_size_t * len(names))(*[a.nbytes for a in arrs])
        if outputs is None:
            _check(_lib.lib().glowb200_device_manager_run_function(self.h, name.encode(), cn, cb, cs, len(names)))
        else:
            cd = (C.c_int * len(names))(*[2 if k in outputs else 1 for k in names])
            _check(_lib.lib().glowb200_device_manager_run_function_io(self.h, name.encode(), cn, cb, cs, cd, len(names)))

    def set_context_count(self, contexts):
        """Execution contexts (own placeholders and activations each) of networks added from now on."""
        _check(_lib.lib().glowb200_device_manager_set_context_count(self.h, int(contexts)))

    def io_buffer(self, shape, dtype):
        """A numpy array over pinned host memory from the device manager (allocateDeviceIOBuffer)."""
        dtype = np.dtype(dtype)
        n = int(np.prod(shape)) * dtype.itemsize
        p = _lib.lib().glowb200_device_manager_allocate_io_buffer(self.h, max(n, 1))
        if not p:
            raise GlowB200Error(RUNTIME_ERROR, _lib.lib().glowb200_last_error().decode())
        buf = (C.c_uint8 * max(n, 1)).from_address(p)
        arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
        self._io.append(p)
        return arr

    def run_function_async(self, name, bindings, outputs=()):
        """Enqueues a request (inputs in, kernels, outputs out on three streams) and returns its
        ticket; the arrays must stay alive and untouched until wait(ticket) has returned."""
        names = list(bindings)
        arrs = [bindings[k] for k in names]
        cn = (C.c_char_p * len(names))(*[k.encode() for k in names])
        cb = (C.c_void_p * len(names))(*[a.ctypes.data for a in arrs])
        cs = (C.c_size_t * len(names))(*[a.nbytes for a in arrs])
        cd = (C.c_int * len(names))(*[2 if k in outputs else 1 for k in names])
        ticket = C.c_int64(0)
        _check(_lib.lib().glowb200_device_manager_run_function_async(self.h, name.encode(), cn, cb, cs, cd, len(names),
                                                                     C.byref(ticket)))
        self._inflight[ticket.value] = (cn, cb, cs, cd, arrs)
        return int(ticket.value)

    def wait(self, ticket):
        try:
            _check(_lib.lib().glowb200_device_manager_wait(self.h, int(ticket)))
        finally:
            self._inflight.pop(ticket, None)

    def placeholder_address(self, name, placeholder):
        """(device address, bytes) of a placeholder of a loaded network (device-resident tensors)."""
        ptr, n = C.c_void_p(), C.c_size_t()
        _check(_lib.lib().glowb200_device_manager_placeholder_address(self.h, name.encode(), placeholder.encode(),
                                                                      C.byref(ptr), C.byref(n)))
        return int(ptr.value), int(n.value)

    def transfer_static_placeholder(self, name, placeholder, array):
        """One host-to-device copy of a placeholder that stays put (an embedding table marked static)."""
        a = np.ascontiguousarray(array)
        _check(_lib.lib().glowb200_device_manager_transfer_static_placeholder(self.h, name.encode(), placeholder.encode(),
                                                                              C.c_void_p(a.ctypes.data), a.nbytes))

    def run_function_resident(self, name):
        """Runs the network on its placeholders as they are in device memory: no copies."""
        _check(_lib.lib().glowb200_device_manager_run_function_resident(self.h, name.encode()))

    @property
    def maximum_memory(self):
        return int(_lib.lib().glowb200_device_manager_maximum_memory(self.h))

    @property
    def available_memory(self):
        return int(_lib.lib().glowb200_device_manager_available_memory(self.h))

    def is_memory_available(self, estimate):
        return bool(_lib.lib().glowb200_device_manager_is_memory_available(self.h, int(estimate)))

    def stop(self):
        _check(_lib.lib().glowb200_device_manager_stop(self.h))
        self._functions.clear()

    def __del__(self):
        if getattr(self, "h", None):
            for p in self._io:
                _lib.lib().glowb200_device_manager_free_io_buffer(self.h, C.c_void_p(p))
            self._io = []
            _lib.lib().glowb200_device_manager_destroy(self.h)
            self.h = None
