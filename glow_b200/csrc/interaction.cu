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
  pdl_wait();               // (launched as a programmatic dependent of the pooling kernel)
  pdl_launch_dependents();  // a contraction that follows may set up now (it waits for this kernel before its loads)
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

// (Measured on B200, 512 and 4096 samples of 65 x 128: this kernel 21 / 138 us.  An 8 x 4 tile
// variant over a transposed copy in shared memory with packed f32x2 FMAs and a staged, coalesced
// result row executed 15 % fewer instructions but ran at half the warps per SM and came out at
// 27 / 138 us: both forms issue about one instruction every other cycle per scheduler, so it is
// latency at low occupancy, not shared-memory bandwidth, that bounds them.)
// The same result from 4 x 4 register tiles (D a multiple of 4): a thread owns the dots of rows
// bi + r*nb against rows bj + s*nb (r, s = 0..3, nb = ceil(n / 4), bj <= bi) and walks k four at a time with 16-byte
// shared-memory loads -- 8 loads feed 64 FMAs instead of 2 loads per FMA, which is what bounded
// the kernel above.  Every dot still is the sequential FMA chain over k = 0..D-1, so the bits are
// the same.  Rows are padded by 4 floats (D + 4, an odd number of 16-byte units for D a multiple of 8) so that
// the neighbouring rows a warp reads fall into different banks.
__global__ void __launch_bounds__(256) pairwise_dot_tiled_kernel(const float *__restrict__ dense, int64_t ld_dense,
                                                                 const float *__restrict__ pooled, int64_t ld_pooled,
                                                                 int tables, int D, float *__restrict__ out_f,
                                                                 int8_t *__restrict__ out_q, int64_t ld_out, float q_scale,
                                                                 int32_t q_offset, int vec_in) {
  pdl_wait();               // (launched as a programmatic dependent of the pooling kernel)
  pdl_launch_dependents();  // a contraction that follows may set up now (it waits for this kernel before its loads)
  extern __shared__ __align__(16) float v[];  // [4 * ceil(n / 4)][D + 4]; rows beyond n are zero
  const int n = tables + 1, pitch = D + 4, nb = (n + 3) >> 2;
  const int64_t b = blockIdx.x;
  if (vec_in) {
    const int q = D >> 2;
    for (int i = threadIdx.x; i < nb * 4 * q; i += blockDim.x) {
      const int r = i / q, k = (i - r * q) * 4;
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < n) x = r == 0 ? __ldg(reinterpret_cast<const float4 *>(dense + b * ld_dense + k))
                            : __ldg(reinterpret_cast<const float4 *>(pooled + b * ld_pooled + (int64_t)(r - 1) * D + k));
      *reinterpret_cast<float4 *>(v + r * pitch + k) = x;
    }
  } else {
    for (int i = threadIdx.x; i < nb * 4 * D; i += blockDim.x) {
      const int r = i / D, k = i - r * D;
      v[r * pitch + k] = r >= n ? 0.0f : (r == 0 ? dense[b * ld_dense + k] : pooled[b * ld_pooled + (int64_t)(r - 1) * D + k]);
    }
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
  const int tiles = nb * (nb + 1) / 2;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    // t -> (bi, bj), bj <= bi, row-major over the lower triangle of tiles
    int bi = (int)((sqrtf(1.0f + 8.0f * (float)t) - 1.0f) * 0.5f);
    while (bi * (bi + 1) / 2 > t) bi--;
    while ((bi + 1) * (bi + 2) / 2 <= t) bi++;
    const int bj = t - bi * (bi + 1) / 2;
    // the tile's rows are bi + r*nb against bj + s*nb (strided, not adjacent): neighbouring
    // threads then read neighbouring rows, which the odd pitch / 4 spreads over all banks
    const float *a = v + bi * pitch, *c = v + bj * pitch;
    const int tile_step = nb * pitch;
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
      for (int s = 0; s < 4; s++) acc[r][s] = 0.0f;
    for (int k = 0; k < D; k += 4) {
      float4 x[4], y[4];
#pragma unroll
      for (int r = 0; r < 4; r++) {
        x[r] = *reinterpret_cast<const float4 *>(a + r * tile_step + k);
        y[r] = *reinterpret_cast<const float4 *>(c + r * tile_step + k);
      }
#pragma unroll
      for (int r = 0; r < 4; r++)
#pragma unroll
        for (int s = 0; s < 4; s++) {
          acc[r][s] = fmaf(x[r].x, y[s].x, acc[r][s]);
          acc[r][s] = fmaf(x[r].y, y[s].y, acc[r][s]);
          acc[r][s] = fmaf(x[r].z, y[s].z, acc[r][s]);
          acc[r][s] = fmaf(x[r].w, y[s].w, acc[r][s]);
        }
    }
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
      for (int s = 0; s < 4; s++) {
        // a dot product is symmetric: the tile of two different residue classes holds every
        // pair between them once; the diagonal tile holds each pair twice and keeps one
        const int i = bi + r * nb, j = bj + s * nb;
        const int hi = i > j ? i : j, lo = i > j ? j : i;
        if (hi < n && lo < hi && (bi != bj || i > j)) emit(D + hi * (hi - 1) / 2 + lo, acc[r][s]);
      }
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
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
  const size_t tiled_smem = (size_t)((n + 3) / 4 * 4) * (dim + 4) * sizeof(float);
  if ((dim % 4) == 0 && tiled_smem <= 200 * 1024) {
    static int raised_for[64];  // largest dynamic shared-memory size enabled so far, per device
    int dev = 0;
    GLOWB200_CUDA_OK(cudaGetDevice(&dev));
    if (tiled_smem > 48 * 1024 && (int)tiled_smem > raised_for[dev & 63]) {
      GLOWB200_CUDA_OK(cudaFuncSetAttribute(pairwise_dot_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tiled_smem));
      raised_for[dev & 63] = (int)tiled_smem;
    }
    const int vec_in = (reinterpret_cast<uintptr_t>(dense) % 16 == 0) && (ld_dense % 4 == 0) &&
                       (tables == 0 || (reinterpret_cast<uintptr_t>(pooled) % 16 == 0 && ld_pooled % 4 == 0));
    GLOWB200_CUDA_OK(launch_pdl(pairwise_dot_tiled_kernel, (unsigned)batch, 256, tiled_smem, cs, dense, ld_dense, pooled, ld_pooled,
                                (int)tables, (int)dim, out_f32, out_i8, ld_out, quant_scale, quant_offset, vec_in));
    return GLOWB200_OK;
  }
  const size_t smem = (size_t)n * (dim + 1) * sizeof(float);
  GLOWB200_REQUIRE(smem <= 200 * 1024, "tables x dim too large for one block's shared memory");
  if (smem > 48 * 1024)
    GLOWB200_CUDA_OK(cudaFuncSetAttribute(pairwise_dot_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  GLOWB200_CUDA_OK(launch_pdl(pairwise_dot_kernel, (unsigned)batch, 256, smem, reinterpret_cast<cudaStream_t>(stream), dense, ld_dense,
                              pooled, ld_pooled, (int)tables, (int)dim, out_f32, out_i8, ld_out, quant_scale, quant_offset));
  return GLOWB200_OK;
}
