// DLRM feature interaction: for every sample, the dot products of all pairs among the bottom-MLP
// output and the pooled embedding vectors, concatenated behind the bottom-MLP output.
//
// The reference builds this from generic nodes -- Concat, Reshape to [B, n, D], BatchMatMul with
// its own transpose, then a flatten (tests/unittests/RecommendationSystemTest.cpp:640-680) -- and
// has no kernel of its own for it.  The benchmark's model keeps only the strictly-lower triangle
// of the n x n product (n = tables + 1, pairs (i, j) with j < i in row-major order, the DLRM
// convention): out[b] = [ v_0 (D values) | v_1.v_0 | v_2.v_0 | v_2.v_1 | v_3.v_0 | ... ].
// One block per sample keeps the n vectors in shared memory; a dot product is a sequential fp32
// FMA chain over the D components.  The result can be written as fp32 or already quantized to
// int8 (Quantize fused: nearbyintf(x / scale + offset), clipped).
#include "common.cuh"

namespace glowb200 {
namespace {

__global__ void __launch_bounds__(256) pairwise_dot_kernel(const float *__restrict__ dense, int64_t ld_dense,
                                                           const float *__restrict__ pooled, int64_t ld_pooled, int tables,
                                                           int D, float *__restrict__ out_f, int8_t *__restrict__ out_q,
                                                           int64_t ld_out, float q_scale, int32_t q_offset) {
  extern __shared__ float v[];  // [n][D + 1]
  const int n = tables + 1, pitch = D + 1;
  const int64_t b = blockIdx.x;
  for (int i = threadIdx.x; i < n * D; i += blockDim.x) {
    const int r = i / D, k = i - r * D;
    v[r * pitch + k] = r == 0 ? dense[b * ld_dense + k] : pooled[b * ld_pooled + (int64_t)(r - 1) * D + k];
  }
  __syncthreads();
  auto emit = [&](int64_t col, float x) {
    if (out_q) {
      const float t = __fadd_rn(__fdiv_rn(x, q_scale), (float)q_offset);
      const float c = fminf(fmaxf(nearbyintf(t), -2147483648.0f), 2147483520.0f);
      out_q[b * ld_out + col] = (int8_t)clip_i8((int32_t)c);
    } else {
      out_f[b * ld_out + col] = x;
    }
  };
  for (int k = threadIdx.x; k < D; k += blockDim.x) emit(k, v[k]);
  const int pairs = n * (n - 1) / 2;
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    // p -> (i, j), j < i, row-major over the strictly-lower triangle
    int i = (int)((1.0f + sqrtf(1.0f + 8.0f * (float)p)) * 0.5f);
    while (i * (i - 1) / 2 > p) i--;
    while ((i + 1) * i / 2 <= p) i++;
    const int j = p - i * (i - 1) / 2;
    const float *a = v + i * pitch, *c = v + j * pitch;
    float acc = 0.0f;
    for (int k = 0; k < D; k++) acc = fmaf(a[k], c[k], acc);
    emit(D + p, acc);
  }
}

}  // namespace
}  // namespace glowb200

using namespace glowb200;

extern "C" int glowb200_pairwise_dot_interaction(const float *dense, int64_t ld_dense, const float *pooled,
                                                 int64_t ld_pooled, int64_t batch, int64_t tables, int64_t dim,
                                                 float *out_f32, int8_t *out_i8, int64_t ld_out, float quant_scale,
                                                 int32_t quant_offset, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(batch >= 0 && tables >= 0 && dim > 0 && tables < 4096 && dim <= 4096 && batch < (1ll << 31),
                   "bad sizes");
  if (batch == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(dense && (tables == 0 || pooled) && ((out_f32 != nullptr) != (out_i8 != nullptr)),
                   "need dense, pooled and exactly one of the two outputs");
  const int64_t n = tables + 1, width = dim + n * (n - 1) / 2;
  GLOWB200_REQUIRE(ld_out >= width && ld_dense >= dim && ld_pooled >= tables * dim, "row pitch smaller than the row");
  const size_t smem = (size_t)n * (dim + 1) * sizeof(float);
  GLOWB200_REQUIRE(smem <= 200 * 1024, "tables x dim too large for one block's shared memory");
  if (smem > 48 * 1024)
    GLOWB200_CUDA_OK(cudaFuncSetAttribute(pairwise_dot_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  pairwise_dot_kernel<<<(unsigned)batch, 256, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      dense, ld_dense, pooled, ld_pooled, (int)tables, (int)dim, out_f32, out_i8, ld_out, quant_scale, quant_offset);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}
