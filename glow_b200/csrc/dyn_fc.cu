// Dynamically quantized fully connected layers: DynamicRowwiseQuantizedFullyConnected and
// DynamicQuantizedFullyConnected.
//
// Reference: fwdDynRowwiseQuantizedFullyConnectedInstPreimpl / ...InstImpl and
// fwdDynamicQuantizedFullyConnectedInst (lib/Backends/Interpreter/InterpreterNodes.cpp:4677-4790;
// the CPU backend has no kernel for these nodes).  Every row of the fp16 input gets its own
// symmetric int8 parameters from its minimum and maximum (chooseQuantizationParams,
// lib/Quantization/Base/Base.cpp:433-565), is quantized with them (quantization::quantize,
// include/glow/Quantization/Base/Base.h:322-329), multiplied with the int8 weights into int32
// sums, and the result is fp16(float(sum) * (row scale * weight scale[j]) + bias[j]).
//
// Two launches: a warp per input row finds the range, derives the parameters in the reference's
// double arithmetic and writes the int8 row, its scale and (for weights with offsets) its sum;
// then the tcgen05 contraction of qgemm.cu runs with its floating-point drain.
#include "qgemm.cuh"
#include "quant_math.cuh"

namespace glowb200 {
namespace {

// quantization::quantize<int8_t> (include/glow/Quantization/Base/Base.h:322-329) with an offset already a float.
__device__ __forceinline__ int32_t quantize_i8(float x, float scale, float offset) {
  const float r = __fadd_rn(__fdiv_rn(x, scale), offset);
  long long v = (long long)rintf(r);
  return (int32_t)(v < -128 ? -128 : (v > 127 ? 127 : v));
}

// in [M, K] fp16 -> q [M, K] int8, row_scales [M], row_sums [M] (may be nullptr).  A block per
// row, element by element: the form for rows that are not 16-byte aligned multiples of 8.
constexpr int kQuantThreads = 256;

__global__ void __launch_bounds__(kQuantThreads) dyn_quantize_rows_kernel(const __half *__restrict__ in, int M, int K,
                                                                          int8_t *__restrict__ q, float *__restrict__ row_scales,
                                                                          int32_t *__restrict__ row_sums, int32_t *status) {
  pdl_launch_dependents();  // a contraction that follows may set up now (it waits for this kernel before its loads)
  __shared__ float s_mn[kQuantThreads / 32], s_mx[kQuantThreads / 32];
  __shared__ int32_t s_sum[kQuantThreads / 32];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const __half *x = in + (size_t)row * K;
  // minMaxArg over the row: NaNs never win a comparison
  float mn = __half2float(x[0]), mx = mn;
  for (int k = tid; k < K; k += kQuantThreads) {
    const float v = __half2float(x[k]);
    mn = v < mn ? v : mn;
    mx = v > mx ? v : mx;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float a = __shfl_xor_sync(0xffffffffu, mn, d), b = __shfl_xor_sync(0xffffffffu, mx, d);
    mn = a < mn ? a : mn;
    mx = b > mx ? b : mx;
  }
  if (lane == 0) { s_mn[warp] = mn; s_mx[warp] = mx; }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kQuantThreads / 32; i++) {
    mn = s_mn[i] < mn ? s_mn[i] : mn;
    mx = s_mx[i] > mx ? s_mx[i] : mx;
  }
  double scale_d;
  int32_t offset;
  choose_quantization_params_basic(mn, mx, /*Symmetric*/ 1, -128, 127, scale_d, offset);
  const float scale = (float)scale_d, foffset = (float)offset;
  // A symmetric range always nudges the zero point to 0; the contraction relies on it.
  if (offset != 0 && tid == 0 && status != nullptr) atomicOr(status, GLOWB200_STATUS_UNSUPPORTED_TABLE);
  int32_t sum = 0;
  int8_t *o = q + (size_t)row * K;
  for (int k = tid; k < K; k += kQuantThreads) {
    const int32_t v = quantize_i8(__half2float(x[k]), scale, foffset);
    o[k] = (int8_t)v;
    sum += v;
  }
  if (row_sums != nullptr) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if (lane == 0) s_sum[warp] = sum;
    __syncthreads();
    if (tid == 0) {
      int32_t total = 0;
      for (int i = 0; i < kQuantThreads / 32; i++) total += s_sum[i];
      row_sums[row] = total;
    }
  }
  if (tid == 0) row_scales[row] = scale;
}

// fp16 bits -> float through the mixed-precision add (adding -0 keeps every value): conversion
// instructions issue at an eighth of the rate.
__device__ __forceinline__ float widen_f16(uint32_t h) {
  float d;
  asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"((uint16_t)(h & 0xFFFFu)), "f"(-0.0f));
  return d;
}

// A WARP per row (K a multiple of 8, 16-byte aligned rows): the range is found on the fp16 pairs
// themselves and reduced with shuffles, the second pass reads the row again (from L1 / L2) so
// that few registers are held and many warps stay resident, and no block-wide barrier sits
// between the load and the store.  Eight elements are quantized by reciprocal at a time; a tie
// candidate among them sends the eight through the exact division.
__global__ void __launch_bounds__(256) dyn_quantize_rows_warp_kernel(const __half *__restrict__ in, int M, int K,
                                                                     int8_t *__restrict__ q, float *__restrict__ row_scales,
                                                                     int32_t *__restrict__ row_sums, int32_t *status) {
  pdl_launch_dependents();  // a contraction that follows may set up now (it waits for this kernel before its loads)
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const __half *x = in + (size_t)row * K;
  // minMaxArg over the row (NaNs never win a comparison; min / max of fp16 numbers is exact)
  __half2 mn2 = __half2half2(x[0]), mx2 = mn2;
#pragma unroll 4
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 v = *reinterpret_cast<const uint4 *>(x + k);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
      mn2 = __hmin2(mn2, h);
      mx2 = __hmax2(mx2, h);
    }
  }
  float mn = fminf(__low2float(mn2), __high2float(mn2)), mx = fmaxf(__low2float(mx2), __high2float(mx2));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, d));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  }
  // Handle::minMaxArg starts from element 0 and keeps what no later element beats: a NaN there
  // stays (every comparison with it is false), a NaN anywhere else never gets in.  The min / max
  // instructions above drop NaNs wherever they are, so the first element is looked at again --
  // the row then quantizes as it does in the kernel that compares with '<' and '>'.
  {
    const float x0 = __half2float(x[0]);
    if (x0 != x0) mn = mx = x0;
  }
  double scale_d;
  int32_t offset;
  choose_quantization_params_basic(mn, mx, /*Symmetric*/ 1, -128, 127, scale_d, offset);
  const float scale = (float)scale_d, foffset = (float)offset;
  const float rcp = __frcp_rn(scale);
  if (offset != 0 && lane == 0 && status != nullptr) atomicOr(status, GLOWB200_STATUS_UNSUPPORTED_TABLE);
  int32_t sum = 0;
  int8_t *o = q + (size_t)row * K;
#pragma unroll 2
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 v = *reinterpret_cast<const uint4 *>(x + k);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      f[2 * i] = widen_f16(w[i]);
      f[2 * i + 1] = widen_f16(w[i] >> 16);
    }
    int32_t r[8];
    bool exact = offset != 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      // x times the row's reciprocal, rounded to the nearest integer by the 1.5 * 2^23 trick, which
      // leaves the integer in the mantissa; within 1e-4 of a tie (the product is within 3e-5 of
      // the true quotient at |quotient| <= 128), or when not small, the exact division decides
      const float p = __fmul_rn(f[i], rcp);
      const float m = __fadd_rn(p, 12582912.0f);
      const float d = fabsf(__fsub_rn(p, __fsub_rn(m, 12582912.0f)));
      exact |= !(d < 0.4999f) || !(fabsf(p) < 1000.0f);
      const int32_t t = __float_as_int(m) - 0x4B400000;
      r[i] = t < -128 ? -128 : (t > 127 ? 127 : t);
    }
    if (exact) {  // (unrolled: a loop would put f and r into local memory)
#pragma unroll
      for (int i = 0; i < 8; i++) r[i] = quantize_i8(f[i], scale, foffset);
    }
    uint32_t packed[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      sum += r[4 * h] + r[4 * h + 1] + r[4 * h + 2] + r[4 * h + 3];
      packed[h] = (uint32_t)(r[4 * h] & 0xff) | ((uint32_t)(r[4 * h + 1] & 0xff) << 8) | ((uint32_t)(r[4 * h + 2] & 0xff) << 16) |
                  ((uint32_t)(r[4 * h + 3] & 0xff) << 24);
    }
    *reinterpret_cast<uint2 *>(o + k) = make_uint2(packed[0], packed[1]);
  }
  if (row_sums != nullptr) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if (lane == 0) row_sums[row] = sum;
  }
  if (lane == 0) row_scales[row] = scale;
}

int run(void *out, const void *in, const int8_t *weights, const float *bias, const float *scales, const int32_t *offsets,
        float u_scale, int32_t u_offset, int64_t M, int64_t K, int64_t N, const int8_t *weights_transposed, int flags,
        void *workspace, size_t workspace_bytes, int32_t *status, cudaStream_t s) {
  GLOWB200_REQUIRE(M >= 0 && N >= 0 && K > 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 24),
                   "matrix dimensions out of range");
  if (M == 0 || N == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(out && in && (weights || weights_transposed) && bias, "NULL tensor pointer");
  const size_t need = glowb200_dynamic_fc_workspace_bytes(M, K, N);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(GLOWB200_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  GLOWB200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  uint8_t *w = reinterpret_cast<uint8_t *>(workspace);
  int8_t *q = reinterpret_cast<int8_t *>(w);
  w += align_up((size_t)M * K, 256);
  float *row_scales = reinterpret_cast<float *>(w);
  w += align_up((size_t)M * 4, 256);
  int32_t *row_sums = reinterpret_cast<int32_t *>(w);
  w += align_up((size_t)M * 4, 256);
  int8_t *wt = reinterpret_cast<int8_t *>(w);
  w += align_up((size_t)N * K, 256);
  const bool offsets_zero = (flags & GLOWB200_FC_WEIGHT_OFFSETS_ZERO) != 0 || (offsets == nullptr && u_offset == 0);
  const bool vec = (K % 8) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0;
  int32_t *sums = offsets_zero ? nullptr : row_sums;
  const __half *x = reinterpret_cast<const __half *>(in);
  if (vec)
    dyn_quantize_rows_warp_kernel<<<(unsigned)((M + 7) / 8), 256, 0, s>>>(x, (int)M, (int)K, q, row_scales, sums, status);
  else
    dyn_quantize_rows_kernel<<<(unsigned)M, kQuantThreads, 0, s>>>(reinterpret_cast<const __half *>(in), (int)M, (int)K, q,
                                                                           row_scales, offsets_zero ? nullptr : row_sums, status);
  GLOWB200_CUDA_OK(cudaGetLastError());
  GemmParams p{};
  p.float_out = 1;
  p.out_f16 = reinterpret_cast<__half *>(out);
  p.row_scales = row_scales;
  p.col_scales = scales;
  p.u_col_scale = u_scale;
  p.bias_f32 = bias;
  p.b_offsets = offsets;
  p.u_b_offset = u_offset;
  p.a_row_sums = offsets_zero ? nullptr : row_sums;
  p.status = status;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.k_corr = (int)K;
  const bool tensor_cores = !(flags & GLOWB200_FC_FORCE_ANY_SHAPE_KERNEL) && (K % 16) == 0;
  if (!tensor_cores && weights != nullptr) return run_gemm_float_any(p, q, weights, s);
  const int8_t *b = weights_transposed;
  if (b == nullptr) {
    if (int rc = transpose_i8(weights, wt, (int)K, (int)N, s)) return rc;
    b = wt;
  }
  const size_t used = (size_t)(w - reinterpret_cast<uint8_t *>(workspace));
  return run_gemm(p, q, b, nullptr, offsets_zero, tensor_cores ? 0 : 1, w, workspace_bytes - used, s);
}

}  // namespace
}  // namespace glowb200

using namespace glowb200;

extern "C" size_t glowb200_dynamic_fc_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  if (M < 0 || N < 0 || K < 0) return 0;
  // quantized input, row scales, row sums, a transposed copy of the weights, the contraction's own
  return align_up((size_t)M * K, 256) + 2 * align_up((size_t)M * 4, 256) + align_up((size_t)N * K, 256) +
         i8_gemm_core_workspace_bytes(M, N);
}

extern "C" int glowb200_dynamic_rowwise_quantized_fc(void *out, const void *in, const int8_t *weights, const float *bias,
                                                      const float *scales, const int32_t *offsets, int64_t M, int64_t K,
                                                      int64_t N, const int8_t *weights_transposed, int flags,
                                                      void *workspace, size_t workspace_bytes, int32_t *status,
                                                      glowb200_stream_t stream) {
  GLOWB200_REQUIRE(N == 0 || M == 0 || (scales != nullptr && offsets != nullptr), "scales / offsets is NULL");
  return run(out, in, weights, bias, scales, offsets, 0.0f, 0, M, K, N, weights_transposed, flags, workspace,
             workspace_bytes, status, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int glowb200_dynamic_quantized_fc(void *out, const void *in, const int8_t *weights, const float *bias,
                                              float weights_scale, int32_t weights_offset, int64_t M, int64_t K, int64_t N,
                                              const int8_t *weights_transposed, int flags, void *workspace,
                                              size_t workspace_bytes, int32_t *status, glowb200_stream_t stream) {
  return run(out, in, weights, bias, nullptr, nullptr, weights_scale, weights_offset, M, K, N, weights_transposed, flags,
             workspace, workspace_bytes, status, reinterpret_cast<cudaStream_t>(stream));
}
