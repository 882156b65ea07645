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

// in [M, K] fp16 -> q [M, K] int8, row_scales [M], row_sums [M] (may be nullptr).
__global__ void __launch_bounds__(256) dyn_quantize_rows_kernel(const __half *__restrict__ in, int M, int K,
                                                                int8_t *__restrict__ q, float *__restrict__ row_scales,
                                                                int32_t *__restrict__ row_sums, int32_t *status) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const __half *x = in + (size_t)row * K;
  // minMaxArg over the row: NaNs never win a comparison
  float mn = __half2float(x[0]), mx = mn;
  for (int k = lane; k < K; k += 32) {
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
  double scale_d;
  int32_t offset;
  choose_quantization_params_basic(mn, mx, /*Symmetric*/ 1, -128, 127, scale_d, offset);
  const float scale = (float)scale_d;
  // A symmetric range always nudges the zero point to 0; the contraction relies on it.
  if (offset != 0 && lane == 0 && status != nullptr) atomicOr(status, GLOWB200_STATUS_UNSUPPORTED_TABLE);
  int32_t sum = 0;
  int8_t *o = q + (size_t)row * K;
  for (int k = lane; k < K; k += 32) {
    const float r = __fadd_rn(__fdiv_rn(__half2float(x[k]), scale), (float)offset);
    long long v = (long long)rintf(r);
    v = v < -128 ? -128 : (v > 127 ? 127 : v);
    o[k] = (int8_t)v;
    sum += (int32_t)v;
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
  dyn_quantize_rows_kernel<<<(unsigned)((M + 7) / 8), 256, 0, s>>>(reinterpret_cast<const __half *>(in), (int)M, (int)K, q,
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
