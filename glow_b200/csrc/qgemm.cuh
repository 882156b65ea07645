// Internal interface of the int8 contraction core (qgemm.cu), shared with the convolution
// front end (conv.cu).
#pragma once
#include "common.cuh"

namespace glowb200 {

struct GemmParams {
  int8_t *out;                // [M, N]
  const int32_t *bias;        // [N] or nullptr (MatMul); int8 values when bias_is_i8 (the _i8_i8 kernels)
  const int32_t *b_offsets;   // weight offsets; index j * stride_b_off
  const int32_t *bias_pre, *bias_post, *bias_scale;  // index j * stride_q
  const int32_t *out_pre, *out_post, *out_scale;      // index j * stride_q
  const int32_t *b_row_sums;  // [N] sum_k B[j,k]
  const int32_t *a_row_sums;  // [M] sum_k A[i,k], or nullptr when every b offset is 0
  int32_t *status;
  const int32_t *bias_offsets;  // per-column bias offsets (channelwise conv), or nullptr: bias_offset
  int M, N, K;                  // K: row pitch of both operands in bytes (a multiple of 16 on the TMA path)
  int k_corr;                   // number of real K entries (<= K; the rest is zero padding); 0 = K
  int32_t a_offset, bias_offset, out_offset;
  // fused activation on the requantised value (glow::FusedActivation: 0 none, 1 relu, 2 clip, 5 leaky relu)
  int32_t act_type, act_args[3];
  // per-tensor layers: one set of scalars for every column instead of the arrays above
  int uniform;
  int bias_is_i8;
  // Shifted-rows convolution (conv_entries > 0; stride 1, no dilation, no groups): the left operand
  // is the padded NHWC input seen as a matrix [padded pixels, C].  Output pixel (n, oh, ow) is row
  // q = (n * Hp + oh) * Wp + ow of the product, and filter tap (kh, kw) reads row q + kh * Wp + kw:
  // k-block kb of a tile starting at row m0 loads rows m0 + conv_row_off[kb / conv_cpb], 128-byte
  // channel block kb % conv_cpb.  Rows whose (oh, ow) fall outside the output are computed and
  // dropped; the result is stored densely as [n, oh, ow, N].
  int conv_entries, conv_cpb;
  // Row-window convolution (conv_windows = windows per plane, != 0; stride 2, few channels -- a stem):
  // the left operand is two planes of 32-byte windows [plane e][n][y][ow], one after the other (the
  // taps (kh = 2a + e, kw = 0..7) of output pixel (n, oh, ow) are window (n, oh + a, ow) of plane e).
  // k-block kb is plane kb: four loads bring windows q + a * conv_wp (a = 0..3) of the tile's 128
  // pixels q as four 128 x 32-byte tiles, one per MMA k-step.  Output pixel (n, oh, ow) is row
  // (n * Y + oh) * OW + ow of the product (conv_hpwp = Y * OW, conv_wp = OW); rows with oh >= conv_oh
  // are computed and dropped.
  int conv_windows;
  int conv_row_off[32];
  int conv_hpwp, conv_wp, conv_oh, conv_ow;
  int32_t u_b_offset, u_bias_pre, u_bias_post, u_bias_scale, u_out_pre, u_out_post, u_out_scale;
  // Floating-point result (dynamically quantized layers; float_out != 0): out_f16[i,j] =
  // fp16(float(sum_ij) * (row_scales[i] * col_scales[j]) + bias_f32[j]), sum_ij the int32 dot
  // product of (A - 0) and (B - b_offsets[j]); every product and the sum are rounded separately.
  // col_scales / b_offsets may be NULL: u_col_scale / u_b_offset for every column.
  int float_out;
  __half *out_f16;
  const float *row_scales, *col_scales, *bias_f32;
  float u_col_scale;
};

struct ColQuant {
  int32_t b_off, bias_pre, bias_post, bias_scale, out_pre, out_post, out_scale;
};
__device__ __forceinline__ ColQuant col_quant(const GemmParams &p, int j) {
  if (p.uniform) return {p.u_b_offset, p.u_bias_pre, p.u_bias_post, p.u_bias_scale, p.u_out_pre, p.u_out_post, p.u_out_scale};
  return {p.b_offsets[j], p.bias ? p.bias_pre[j] : 0, p.bias ? p.bias_post[j] : 0, p.bias ? p.bias_scale[j] : 0,
          p.out_pre[j], p.out_post[j], p.out_scale[j]};
}

// bias[j] of either element type (libjit_fc_generic / libjit_rowwise_quantized_fc_generic /
// libjit_*_conv2d_generic are templates over BiasElemTy: int32 for the _i8_i32 entry points, int8 for _i8_i8).
__device__ __forceinline__ int32_t load_bias(const GemmParams &p, int j) {
  return p.bias_is_i8 ? (int32_t) reinterpret_cast<const int8_t *>(p.bias)[j] : p.bias[j];
}

// libjit_activation_i32 (lib/LLVMIRCodeGen/libjit/libjit_defs.h:206-233).
__device__ __forceinline__ int32_t activation_i32(int32_t x, const GemmParams &p) {
  if (p.act_type == 0) return x;
  if (p.act_type == 1) return x > p.out_offset ? x : p.out_offset;
  if (p.act_type == 2) { const int32_t t = x > p.act_args[0] ? x : p.act_args[0]; return t < p.act_args[1] ? t : p.act_args[1]; }
  if (p.act_type == 3 || p.act_type == 4) return x;
  return x >= p.out_offset ? x : scale32(x - p.out_offset, p.act_args[0], p.act_args[1], p.act_args[2], p.out_offset);
}

// out = requant(A[M,K] x B[N,K]^T) with the tensor-core kernel when the shapes allow it (K a
// multiple of 16, 16-byte aligned operands), else the any-shape kernel.  `ws` must hold
// i8_gemm_core_workspace_bytes(M, N) bytes.  b_row_sums_in may be nullptr (computed here).
int run_gemm(GemmParams p, const int8_t *a, const int8_t *b, const int32_t *b_row_sums_in, bool b_offsets_zero,
             int force_any, void *ws, size_t ws_bytes, cudaStream_t s);

// The shifted-rows convolution on the same kernel: `padded` holds `rows` padded pixels of `C` bytes
// (plus 128 readable bytes behind them), p.conv_* describe the taps, p.M = rows, p.K = bytes of a
// row of b (a multiple of 128).  Weight offsets must all be zero (no input row sums).
// buffer_rows: rows the padded buffer holds when the taps reach beyond `rows` (several planes); 0 = rows.
int run_gemm_shifted_rows(GemmParams p, const int8_t *padded, int64_t rows, int C, const int8_t *b,
                          const int32_t *b_row_sums, cudaStream_t s, int64_t buffer_rows = 0);

// The float-result contraction for any shape with the weights in their [K, N] form.
int run_gemm_float_any(const GemmParams &p, const int8_t *a, const int8_t *b_kn, cudaStream_t s);
// [R, C] int8 -> [C, R] int8
int transpose_i8(const int8_t *in_rc, int8_t *out_cr, int R, int C, cudaStream_t s);

// The row-window convolution: `planes` holds two planes of `rows` 32-byte windows each, back to back,
// with 3 * ow + 1 readable windows behind the second; b is [N, 256] (plane, a, 32 bytes).
int run_gemm_row_windows(GemmParams p, const int8_t *planes, int64_t rows, int ow, const int8_t *b, const int32_t *b_row_sums,
                         cudaStream_t s);

inline size_t i8_gemm_core_workspace_bytes(int64_t M, int64_t N) {
  return align_up((size_t)N * 4, 256) + align_up((size_t)M * 4, 256);
}

}  // namespace glowb200
