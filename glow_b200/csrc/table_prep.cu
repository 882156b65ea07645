// Embedding-table preparation and the partial-sum reduction of row-range sharded tables.
#include "common.cuh"
#include "quant_math.cuh"

namespace glowb200 {
namespace {

// tensorFusedRowwiseQuantization<T> (include/glow/Quantization/Base/Base.h:598-678) with
// quantizeWithFloatOffset / quantize4BitsWithFloatOffset (:361-379).  One warp per row: the
// row's minimum and maximum, scale = (max - min) / range computed in double and rounded to
// fp32 (1 when the range is below 1e-10), offset = min; every value is quantized with the fp32
// scale and offset (also for the fp16 kinds, which only STORE them rounded to fp16); 4-bit
// values are clamped to [0, 15] and packed low nibble first.
__global__ void __launch_bounds__(256) fused_rowwise_quantize_kernel(const float *__restrict__ in, int64_t rows,
                                                                      int64_t cols, int kind, uint8_t *__restrict__ out,
                                                                      int64_t out_line) {
  const int lane = threadIdx.x & 31;
  const bool four = kind == GLOWB200_UINT4_FUSED || kind == GLOWB200_UINT4_FUSED_FP16;
  const bool so16 = kind == GLOWB200_UINT8_FUSED_FP16 || kind == GLOWB200_UINT4_FUSED_FP16;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * 8) {
    const float *src = in + row * cols;
    uint8_t *dst = out + row * out_line;
    float mn = src[0], mx = src[0];
    for (int64_t j = lane; j < cols; j += 32) {
      const float v = src[j];
      mn = v < mn ? v : mn;
      mx = v > mx ? v : mx;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float a = __shfl_xor_sync(0xffffffffu, mn, d), b = __shfl_xor_sync(0xffffffffu, mx, d);
      mn = a < mn ? a : mn;
      mx = b > mx ? b : mx;
    }
    const float range = four ? 15.0f : 255.0f;
    const float scale = (__fsub_rn(mx, mn) < 1e-10f) ? 1.0f : (float)(((double)mx - (double)mn) / (double)range);
    const float offset = mn;
    if (!four) {
      for (int64_t j = lane; j < cols; j += 32) {
        const float r = roundf(__fdiv_rn(__fsub_rn(src[j], offset), scale));
        dst[j] = (uint8_t)(uint16_t)r;
      }
    } else {
      for (int64_t b = lane; b < cols / 2; b += 32) {
        int q[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int v = (int)roundf(__fdiv_rn(__fsub_rn(src[2 * b + h], offset), scale));
          q[h] = v < 0 ? 0 : (v > 15 ? 15 : v);
        }
        dst[b] = (uint8_t)(q[0] | (q[1] << 4));
      }
    }
    // scale then offset behind the payload, byte by byte (rows have no alignment to rely on)
    uint64_t packed;
    int tail_bytes;
    if (so16) {
      packed = (uint64_t)__half_as_ushort(__float2half_rn(scale)) | ((uint64_t)__half_as_ushort(__float2half_rn(offset)) << 16);
      tail_bytes = 4;
    } else {
      packed = (uint64_t)__float_as_uint(scale) | ((uint64_t)__float_as_uint(offset) << 32);
      tail_bytes = 8;
    }
    if (lane < tail_bytes) dst[out_line - tail_bytes + lane] = (uint8_t)(packed >> (8 * lane));
  }
}

// One warp per row: payload bytes, zero padding, the scale/offset pair at the end.
__global__ void __launch_bounds__(256) fused_rows_pad_kernel(const uint8_t *__restrict__ src, int64_t rows, int in_line,
                                                              int tail, uint8_t *__restrict__ dst, int padded) {
  const int lane = threadIdx.x & 31;
  const int payload = in_line - tail;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * 8) {
    const uint8_t *s = src + row * in_line;
    uint8_t *d = dst + row * padded;
    for (int j = lane; j < padded; j += 32) {
      uint8_t v = 0;
      if (j < payload) v = s[j];
      else if (j >= padded - tail) v = s[payload + (j - (padded - tail))];
      d[j] = v;
    }
  }
}

// dest[i] = cast(partials[0][i] + partials[1][i] + ...), added in slab order.
template <bool OUT16>
__global__ void __launch_bounds__(256) sum_partials_kernel(const float *__restrict__ partials, int num, int64_t stride,
                                                            int64_t n, void *__restrict__ dest, int vec) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  const int64_t n4 = vec ? (n >> 2) : 0;  // 16-byte path only when every slab and dest allow it
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += step) {
    float4 a = __ldg(reinterpret_cast<const float4 *>(partials) + i);
    for (int g = 1; g < num; g++) {
      const float4 b = __ldg(reinterpret_cast<const float4 *>(partials + g * stride) + i);
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    if constexpr (OUT16) {
      __half2 h[2] = {__floats2half2_rn(a.x, a.y), __floats2half2_rn(a.z, a.w)};
      reinterpret_cast<uint2 *>(dest)[i] = *reinterpret_cast<const uint2 *>(h);
    } else {
      reinterpret_cast<float4 *>(dest)[i] = a;
    }
  }
  for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    float a = partials[i];
    for (int g = 1; g < num; g++) a += partials[g * stride + i];
    if constexpr (OUT16) reinterpret_cast<__half *>(dest)[i] = __float2half_rn(a);
    else reinterpret_cast<float *>(dest)[i] = a;
  }
}

}  // namespace
}  // namespace glowb200

using namespace glowb200;

extern "C" int glowb200_fused_rowwise_quantize_device(const float *in, int64_t rows, int64_t cols, int kind, uint8_t *out,
                                                       int64_t out_line_size, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(kind >= 0 && kind <= 3, "unknown fused kind %d", kind);
  GLOWB200_REQUIRE(rows >= 0 && cols > 0, "rows / cols out of range");
  const bool four = kind >= 2;
  GLOWB200_REQUIRE(!four || cols % 2 == 0, "4-bit fused quantization needs an even number of columns");
  const int64_t want = (four ? cols / 2 : cols) + ((kind & 1) ? 4 : 8);
  GLOWB200_REQUIRE(out_line_size == want, "out_line_size must be %lld for %lld columns of kind %d", (long long)want,
                   (long long)cols, kind);
  if (rows == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(in != nullptr && out != nullptr, "NULL tensor pointer");
  const int64_t want_blocks = (rows + 7) / 8, cap = (int64_t)sm_count() * 16;
  fused_rowwise_quantize_kernel<<<(unsigned)(want_blocks < cap ? want_blocks : cap), 256, 0,
                                  reinterpret_cast<cudaStream_t>(stream)>>>(in, rows, cols, kind, out, out_line_size);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

namespace glowb200 {
namespace {
// quantization::quantize<int8_t> (include/glow/Quantization/Base/Base.h:322-329)
__device__ __forceinline__ int8_t quantize_to_i8(float x, float scale, int32_t offset) {
  const float r = __fadd_rn(__fdiv_rn(x, scale), (float)offset);
  long long v = (long long)rintf(r);
  return (int8_t)(v < -128 ? -128 : (v > 127 ? 127 : v));
}

// tensorRowwiseQuantization<float, int32_t, int8_t> (Base.h:522-576): a block per row finds the
// range, thread 0 derives the parameters (chooseQuantizationParams in the reference's double
// arithmetic), all threads quantize.  given != 0: the parameters are inputs (quantizeTensor with
// per-row parameters, lib/Quantization/Base/Base.cpp:760-777) and only the last step runs.
__global__ void __launch_bounds__(256) rowwise_quantize_i8_kernel(const float *__restrict__ in, long long cols, int schema,
                                                                  int given, int8_t *__restrict__ out, float *scales,
                                                                  int32_t *offsets) {
  __shared__ float s_mn[8], s_mx[8];
  __shared__ float s_scale;
  __shared__ int32_t s_offset;
  const long long row = blockIdx.x;
  const float *x = in + row * cols;
  if (!given) {
    float mn = x[0], mx = mn;
    for (long long k = threadIdx.x; k < cols; k += 256) {
      const float v = x[k];
      mn = v < mn ? v : mn;
      mx = v > mx ? v : mx;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float a = __shfl_xor_sync(0xffffffffu, mn, d), b = __shfl_xor_sync(0xffffffffu, mx, d);
      mn = a < mn ? a : mn;
      mx = b > mx ? b : mx;
    }
    if ((threadIdx.x & 31) == 0) { s_mn[threadIdx.x >> 5] = mn; s_mx[threadIdx.x >> 5] = mx; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < 8; i++) {
        mn = s_mn[i] < mn ? s_mn[i] : mn;
        mx = s_mx[i] > mx ? s_mx[i] : mx;
      }
      double scale;
      int32_t offset;
      choose_quantization_params_basic(mn, mx, schema, -128, 127, scale, offset);
      if (schema == 3) {  // the next power of two at or above the scale: exp2(ceil(log2(scale)))
        int e;
        const double m = frexp(scale, &e);
        scale = ldexp(1.0, m == 0.5 ? e - 1 : e);
      }
      s_scale = (float)scale;
      s_offset = offset;
      scales[row] = (float)scale;
      offsets[row] = offset;
    }
  } else if (threadIdx.x == 0) {
    s_scale = scales[row];
    s_offset = offsets[row];
  }
  __syncthreads();
  const float scale = s_scale;
  const int32_t offset = s_offset;
  for (long long k = threadIdx.x; k < cols; k += 256) out[row * cols + k] = quantize_to_i8(x[k], scale, offset);
}
}  // namespace
}  // namespace glowb200

extern "C" int glowb200_tensor_rowwise_quantize_i8_device(const float *in, int64_t rows, int64_t cols, int schema, int8_t *out,
                                                           float *scales, int32_t *offsets, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(rows >= 0 && rows < (1ll << 31) && cols > 0 && schema >= 0 && schema <= 3, "bad rows / cols / schema");
  if (rows == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(in && out && scales && offsets, "NULL tensor pointer");
  rowwise_quantize_i8_kernel<<<(unsigned)rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(in, cols, schema, 0, out,
                                                                                               scales, offsets);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

extern "C" int glowb200_quantize_rows_i8_device(const float *in, int64_t rows, int64_t cols, const float *scales,
                                                 const int32_t *offsets, int8_t *out, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(rows >= 0 && rows < (1ll << 31) && cols > 0, "bad rows / cols");
  if (rows == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(in && out && scales && offsets, "NULL tensor pointer");
  rowwise_quantize_i8_kernel<<<(unsigned)rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      in, cols, 0, 1, out, const_cast<float *>(scales), const_cast<int32_t *>(offsets));
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

extern "C" int glowb200_fused_rows_pad(const uint8_t *src, int64_t rows, int64_t in_line_size, int64_t tail_bytes,
                                        uint8_t *dst, int64_t padded_line_size, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(tail_bytes == 4 || tail_bytes == 8, "tail_bytes must be 4 or 8");
  GLOWB200_REQUIRE(rows >= 0 && in_line_size > tail_bytes && padded_line_size >= in_line_size && padded_line_size < (1 << 30),
                   "rows / line sizes out of range");
  if (rows == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(src != nullptr && dst != nullptr, "NULL tensor pointer");
  const int64_t want_blocks = (rows + 7) / 8, cap = (int64_t)sm_count() * 32;
  fused_rows_pad_kernel<<<(unsigned)(want_blocks < cap ? want_blocks : cap), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      src, rows, (int)in_line_size, (int)tail_bytes, dst, (int)padded_line_size);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

extern "C" int glowb200_sum_partials(const float *partials, int64_t num_partials, int64_t partial_stride, int64_t n,
                                      void *dest, int dest_is_fp16, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(num_partials >= 1 && num_partials <= 1024 && n >= 0 && partial_stride >= n, "num_partials / n / stride out of range");
  if (n == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(partials != nullptr && dest != nullptr, "NULL tensor pointer");
  const int vec = reinterpret_cast<uintptr_t>(partials) % 16 == 0 && partial_stride % 4 == 0 &&
                  reinterpret_cast<uintptr_t>(dest) % (dest_is_fp16 ? 8 : 16) == 0;
  const int64_t want = (n / 4 + 255) / 256 + 1, cap = (int64_t)sm_count() * 8;
  const unsigned blocks = (unsigned)(want < cap ? want : cap);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dest_is_fp16) sum_partials_kernel<true><<<blocks, 256, 0, s>>>(partials, (int)num_partials, partial_stride, n, dest, vec);
  else sum_partials_kernel<false><<<blocks, 256, 0, s>>>(partials, (int)num_partials, partial_stride, n, dest, vec);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}
