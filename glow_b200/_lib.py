"""ctypes binding of glow_b200/lib/libglow_b200.so (the C ABI of include/glow_b200.h).

There is no fallback: if the CUDA library has not been built, importing an operator raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# GLOW_B200_LIBRARY selects another build of the same library (e.g. one compiled with
# different tuning macros); the default is the in-tree build.
LIB_PATH = os.environ.get("GLOW_B200_LIBRARY") or os.path.join(_HERE, "lib", "libglow_b200.so")

_vp, _i64, _i32, _int, _sz, _f32 = C.c_void_p, C.c_int64, C.c_int32, C.c_int, C.c_size_t, C.c_float


class SlwsJob(C.Structure):
    """struct glowb200_slws_job"""
    _fields_ = [("data", _vp), ("weights", _vp), ("indices", _vp), ("lengths", _vp), ("dest", _vp),
                ("rows", _i64), ("num_indices", _i64), ("dest_stride", _i64), ("segments", _i64),
                ("dests", _vp), ("bags_per_dest", _i64), ("row_begin", _i64), ("global_rows", _i64)]


# name -> (restype, argtypes); also the list the symbol-export test walks.
SIGNATURES = {
    "glowb200_last_error": (C.c_char_p, []),
    "glowb200_version": (C.c_char_p, []),
    "glowb200_slws_workspace_bytes": (_sz, [_i64, _i64]),
    "glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum": (
        _int, [_vp, _vp, _int, _i64, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _int, _int, _vp, _sz, _vp, _vp]),
    "glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_low_latency": (
        _int, [_vp, _vp, _int, _i64, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _int, _vp, _sz, _vp, _vp]),
    "glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_batched": (
        _int, [_vp, _i64, _i64, _int, _int, _i64, _i64, _int, _int, _vp, _sz, _vp, _vp]),
    "glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_row_sharded": (
        _int, [_vp, _i64, _i64, _int, _int, _i64, _i64, _vp, _sz, _vp, _vp]),
    "glowb200_slws_static_scratch_max_segments": (_i64, []),
    "glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_static_scratch": (
        _int, [_vp, _vp, _int, _i64, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _int, _int, _vp, _vp]),
    "glowb200_sparse_lengths_weighted_sum_f32": (
        _int, [_vp, _vp, _i64, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp, _sz, _vp, _vp]),
    "glowb200_rowwise_quantized_sparse_lengths_weighted_sum_f32": (
        _int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp, _sz, _vp, _vp]),
    "glowb200_fused_rowwise_quantize": (_int, [_vp, _i64, _i64, _int, _vp, _i64]),
    "glowb200_fused_rowwise_quantize_device": (_int, [_vp, _i64, _i64, _int, _vp, _i64, _vp]),
    "glowb200_fused_rows_pad": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _vp]),
    "glowb200_sum_partials": (_int, [_vp, _i64, _i64, _i64, _vp, _int, _vp]),
    "glowb200_quantize_scale_offset_32to8": (None, [_f32, _vp, _vp, _vp]),
    "glowb200_rowwise_requant_params": (_int, [_vp, _i64, _f32, _vp, _i64, _f32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "glowb200_choose_quantization_params": (None, [_f32, _f32, _int, _int, _vp, _vp]),
    "glowb200_tensor_rowwise_quantize_i8": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "glowb200_quantize_bias_i32": (_int, [_vp, _i64, _f32, _i32, _vp]),
    "glowb200_channelwise_conv_prepare": (_int, [_vp, _vp, _i64, _i64, _f32, _int] + [_vp] * 6),
    "glowb200_wait_limit_selftest": (_int, [_i64, _vp, _vp, _vp]),
    "glowb200_i8_mma_issue_probe": (_int, [_i64, _vp, _vp, _vp]),
    "glowb200_i8_gemm_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "glowb200_i8_row_sums": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "glowb200_rowwise_quantized_fc_i8_i32": (
        _int, [_vp] * 11 + [_i64, _i64, _i64, _i32, _i32, _i32, _vp, _int, _vp, _sz, _vp, _vp]),
    "glowb200_fc_i8_i32": (
        _int, [_vp] * 4 + [_i64] * 3 + [_i32] * 10 + [_vp, _int, _vp, _sz, _vp, _vp]),
    "glowb200_matmul_i8": (
        _int, [_vp] * 3 + [_i64] * 3 + [_i32] * 6 + [_int, _vp, _sz, _vp, _vp]),
    "glowb200_conv2d_workspace_bytes": (_sz, [_vp] * 6 + [_i64, _vp]),
    "glowb200_channelwise_quantized_conv2d_i8_i32": (
        _int, [_vp] * 10 + [_i64, _vp, _i32, _i32] + [_vp] * 8 + [_i32, _vp, _vp, _int, _vp, _sz, _vp, _vp]),
    "glowb200_conv2d_i8_i32": (
        _int, [_vp] * 10 + [_i64] + [_i32] * 10 + [_vp, _i32, _vp, _int, _vp, _sz, _vp, _vp]),
    "glowb200_element_add_i8": (_int, [_vp, _vp, _vp, _i64] + [_i32] * 9 + [_vp]),
    "glowb200_element_add_maxsplat_i8": (_int, [_vp, _vp, _vp, _i64] + [_i32] * 10 + [_vp]),
    "glowb200_element_binary_i8": (_int, [_int, _vp, _vp, _vp, _i64] + [_i32] * 9 + [_vp]),
    "glowb200_element_muldiv_i8": (_int, [_int, _vp, _vp, _vp, _i64] + [_i32] * 6 + [_vp]),
    "glowb200_batched_add_i8": (_int, [_vp, _vp, _vp, _int, _i64, _i64] + [_i32] * 9 + [_vp]),
    "glowb200_element_relu_i8": (_int, [_vp, _vp, _i64] + [_i32] * 5 + [_vp]),
    "glowb200_element_maxsplat_i8": (_int, [_vp, _vp, _i64, _i32, _vp]),
    "glowb200_splat_f": (_int, [_vp, _i64, _f32, _int, _vp]),
    "glowb200_element_rescale_i8": (_int, [_vp, _vp, _i64] + [_i32] * 5 + [_vp]),
    "glowb200_element_quantize_i8": (_int, [_vp, _vp, _i64, _f32, _i32, _vp]),
    "glowb200_element_dequantize_i8": (_int, [_vp, _vp, _i64, _f32, _i32, _vp]),
    "glowb200_max_pool_i8": (_int, [_vp] * 7 + [_i32, _vp]),
    "glowb200_avg_pool_i8": (_int, [_vp] * 7 + [_int] + [_i32] * 5 + [_vp]),
    "glowb200_transpose": (_int, [_vp, _vp, _vp, _vp, _int, _int, _vp]),
    "glowb200_set_programmatic_launch": (_int, [_int]),
    "glowb200_quantize_transpose_i8": (_int, [_vp, _vp, _vp, _vp, _int, _f32, _i32, _vp]),
    "glowb200_pairwise_dot_interaction": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _i64, _f32, _i32, _vp]),
    "glowb200_peer_buffer_create": (_int, [_sz, _vp, _vp]),
    "glowb200_peer_buffer_open": (_int, [_vp, _vp]),
    "glowb200_peer_buffer_close": (_int, [_vp]),
    "glowb200_peer_buffer_destroy": (_int, [_vp]),
    "glowb200_peer_rendezvous": (_int, [_vp, _vp, _int, _int, _i64, _vp, _vp]),
    "glowb200_function_create": (_vp, [C.c_char_p]),
    "glowb200_function_destroy": (None, [_vp]),
    "glowb200_function_add_symbol": (_int, [_vp, C.c_char_p, _int, _sz, _vp]),
    "glowb200_function_add_instruction": (_int, [_vp, _int, _vp, _int, _vp, _int, _vp, _int]),
    "glowb200_function_batched_pooling_launches": (_int, [_vp]),
    "glowb200_function_fused_quantize_transposes": (_int, [_vp]),
    "glowb200_function_add_instruction_views": (_int, [_vp, _int, _vp, _vp, _int, _vp, _int, _vp, _int]),
    "glowb200_function_compile": (_int, [_vp]),
    "glowb200_function_constant_bytes": (_sz, [_vp]),
    "glowb200_device_manager_create": (_vp, [_int, C.c_uint64]),
    "glowb200_device_manager_init": (_int, [_vp]),
    "glowb200_device_manager_add_network": (_int, [_vp, _vp]),
    "glowb200_device_manager_evict_network": (_int, [_vp, C.c_char_p]),
    "glowb200_device_manager_run_function": (_int, [_vp, C.c_char_p, _vp, _vp, _vp, _int]),
    "glowb200_device_manager_run_function_io": (_int, [_vp, C.c_char_p, _vp, _vp, _vp, _vp, _int]),
    "glowb200_device_manager_set_context_count": (_int, [_vp, _int]),
    "glowb200_device_manager_run_function_async": (_int, [_vp, C.c_char_p, _vp, _vp, _vp, _vp, _int, _vp]),
    "glowb200_device_manager_wait": (_int, [_vp, _i64]),
    "glowb200_device_manager_allocate_io_buffer": (_vp, [_vp, C.c_size_t]),
    "glowb200_device_manager_free_io_buffer": (None, [_vp, _vp]),
    "glowb200_device_manager_placeholder_address": (_int, [_vp, C.c_char_p, C.c_char_p, _vp, _vp]),
    "glowb200_device_manager_transfer_static_placeholder": (_int, [_vp, C.c_char_p, C.c_char_p, _vp, _sz]),
    "glowb200_device_manager_run_function_resident": (_int, [_vp, C.c_char_p]),
    "glowb200_device_manager_maximum_memory": (C.c_uint64, [_vp]),
    "glowb200_device_manager_available_memory": (C.c_uint64, [_vp]),
    "glowb200_device_manager_is_memory_available": (_int, [_vp, C.c_uint64]),
    "glowb200_device_manager_stop": (_int, [_vp]),
    "glowb200_device_manager_destroy": (None, [_vp]),
    "glowb200_embedding_bag_byte_rowwise_offsets": (
        _int, [_vp, _vp, _int, _i64, _vp, _vp, _vp, _int, _i64, _i64, _i64, _i64, _int, _int, _int, _vp, _sz, _vp,
               _vp]),
    "glowb200_tensor_rowwise_quantize_i8_device": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp]),
    "glowb200_quantize_rows_i8_device": (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    "glowb200_quantization_profile_workspace_bytes": (_sz, [_i64]),
    "glowb200_quantization_profile": (_int, [_vp, _i64, _vp, _vp, _i64, _vp, _sz, _vp]),
    "glowb200_dynamic_fc_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "glowb200_dynamic_rowwise_quantized_fc": (
        _int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _int, _vp, _sz, _vp, _vp]),
    "glowb200_dynamic_quantized_fc": (
        _int, [_vp, _vp, _vp, _vp, _f32, _i32, _i64, _i64, _i64, _vp, _int, _vp, _sz, _vp, _vp]),
    "glowb200_int_nbit_split_embedding_bags": (
        _int, [_vp, _vp, _i64, _vp, _i64, _vp, _vp, _int, _vp, _vp, _i64, _i64, _vp, _vp, _int, _i64, _i64, _int,
               _vp, _int, _int, _int, _int, _vp, _vp]),
}

_lib = None


class GlowB200Error(RuntimeError):
    def __init__(self, code, message):
        super().__init__("glow_b200 error %d: %s" % (code, message))
        self.code = code


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with `python -m glow_b200.build` "
                              "(there is no CPU fallback)" % LIB_PATH)
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def check(rc):
    if rc != 0:
        raise GlowB200Error(rc, lib().glowb200_last_error().decode())
