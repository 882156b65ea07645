// The int8 glue operators of a quantized network: element-wise add / relu / max-with-constant
// / rescale, quantize, dequantize, max- and average-pooling, and NCHW <-> NHWC transposes.
// All of them stream their operands once; each kernel restates one libjit kernel.
#include "common.cuh"

namespace glowb200 {
namespace {

constexpr int kThreads = 256;

inline unsigned grid_for(int64_t work_items) {
  const int64_t blocks = (work_items + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  return (unsigned)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

struct Triple { int32_t pre, post, scale; };

// ------------------------------------------------------------------------------------------
// Element-wise int8 kernels.  Each operator is a functor holding its constants; one kernel
// applies it sixteen elements per thread (16-byte loads and stores, when all tensors start on
// 16-byte boundaries) and finishes the tail -- or does everything, for unaligned tensors --
// one element at a time.  These kernels only stream memory: a byte per thread, as they were
// first written, reached a third of the copy bandwidth on a residual block's Add.
// ------------------------------------------------------------------------------------------
// libjit_element_add_kernel_i8 (DEFINE_DATA_PARALLEL_KERNEL_QUANTIZED, libjit.cpp:1593-1603),
// optionally followed by libjit_element_maxsplat_kernel_i8 on its result (the Add and the int8
// Relu of a residual block in one pass over memory).
struct AddF {
  int32_t dst_off, lhs_off, rhs_off;
  Triple lt, rt;
  int32_t splat;  // -128: no max-with-constant behind the add
  __device__ __forceinline__ int32_t operator()(int32_t a, int32_t b) const {
    const int32_t l = scale32(a - lhs_off, lt.pre, lt.post, lt.scale, 0);
    const int32_t r = scale32(b - rhs_off, rt.pre, rt.post, rt.scale, 0);
    const int32_t v = clip_i8(l + r + dst_off);
    return v > splat ? v : splat;
  }
};

// The other arithmetic mini-kernels of DEFINE_DATA_PARALLEL_KERNEL_QUANTIZED (libjit.cpp:1593-1603,
// 1675-1682): both sides rescaled to the result's scale, then sub / max / min, offset, clip.
// OP 1 sub, 2 max, 3 min.
template <int OP>
struct BinaryF {
  int32_t dst_off, lhs_off, rhs_off;
  Triple lt, rt;
  __device__ __forceinline__ int32_t operator()(int32_t a, int32_t b) const {
    const int32_t l = scale32(a - lhs_off, lt.pre, lt.post, lt.scale, 0);
    const int32_t r = scale32(b - rhs_off, rt.pre, rt.post, rt.scale, 0);
    const int32_t v = OP == 1 ? (int32_t)((uint32_t)l - (uint32_t)r) : OP == 2 ? (l > r ? l : r) : (l < r ? l : r);
    return clip_i8((int32_t)((uint32_t)v + (uint32_t)dst_off));
  }
};

// libjit_element_mul_kernel_i8 / _div_kernel_i8 (DEFINE_DATA_PARALLEL_KERNEL_QUANTIZED_M,
// libjit.cpp:1610-1619, 1683-1684): the product (quotient) of the offset-free operands, one
// rescale with the result's offset, clip.  A zero divisor gives the result offset (the
// reference divides by it).
template <bool DIV>
struct MulDivF {
  int32_t dst_off, lhs_off, rhs_off;
  Triple t;
  __device__ __forceinline__ int32_t operator()(int32_t a, int32_t b) const {
    const int32_t l = a - lhs_off, r = b - rhs_off;
    const int32_t v = DIV ? (r == 0 ? 0 : l / r) : (int32_t)((uint32_t)l * (uint32_t)r);
    return clip_i8(scale32(v, t.pre, t.post, t.scale, dst_off));
  }
};

// libjit_element_relu_i8 (libjit.cpp:1850-1858): max(x, srcOffset), then rescale
struct ReluF {
  int32_t src_off, dst_off;
  Triple t;
  __device__ __forceinline__ int32_t operator()(int32_t a, int32_t) const {
    const int32_t v = a > src_off ? a : src_off;
    return clip_i8(scale32(v - src_off, t.pre, t.post, t.scale, dst_off));
  }
};

// libjit_element_maxsplat_kernel_i8 (lib/Backends/CPU/libjit_cpu/libjit_cpu.cpp:39-44)
struct MaxSplatF {
  int32_t splat;
  __device__ __forceinline__ int32_t operator()(int32_t a, int32_t) const { return a > splat ? a : splat; }
};

// libjit_element_rescale_kernel_i8 (libjit.cpp:3030-3038)
struct RescaleF {
  int32_t out_off, in_off;
  Triple t;
  __device__ __forceinline__ int32_t operator()(int32_t a, int32_t) const {
    return clip_i8(scale32(a - in_off, t.pre, t.post, t.scale, out_off));
  }
};

template <typename F>
__device__ __forceinline__ uint32_t map_word(uint32_t a, uint32_t b, const F &f) {
  uint32_t o = 0;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int32_t x = (int32_t)(int8_t)(a >> (8 * j)), y = (int32_t)(int8_t)(b >> (8 * j));
    o |= ((uint32_t)f(x, y) & 0xFFu) << (8 * j);
  }
  return o;
}

// dst[i] = f(lhs[i], rhs[i]) (rhs may be NULL: f ignores its second argument).  vec: all three
// pointers are 16-byte aligned.
template <typename F>
__global__ void __launch_bounds__(kThreads) map_i8_kernel(int8_t *__restrict__ dst, const int8_t *__restrict__ lhs,
                                                          const int8_t *__restrict__ rhs, int64_t n, int vec, const F f) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t nv = vec ? (n >> 4) : 0;
  for (int64_t i = tid; i < nv; i += stride) {
    const uint4 a = __ldg(reinterpret_cast<const uint4 *>(lhs) + i);
    const uint4 b = rhs ? __ldg(reinterpret_cast<const uint4 *>(rhs) + i) : make_uint4(0u, 0u, 0u, 0u);
    uint4 o;
    o.x = map_word(a.x, b.x, f);
    o.y = map_word(a.y, b.y, f);
    o.z = map_word(a.z, b.z, f);
    o.w = map_word(a.w, b.w, f);
    reinterpret_cast<uint4 *>(dst)[i] = o;
  }
  for (int64_t i = (nv << 4) + tid; i < n; i += stride) dst[i] = (int8_t)f((int32_t)lhs[i], rhs ? (int32_t)rhs[i] : 0);
}

template <typename F>
cudaError_t launch_map(int8_t *dst, const int8_t *lhs, const int8_t *rhs, int64_t n, const F &f, cudaStream_t s) {
  const int vec = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) & 15u) == 0;
  if (cudaError_t e = launch_pdl(map_i8_kernel<F>, grid_for(vec ? (n + 15) / 16 : n), kThreads, 0, s, dst, lhs, rhs, n, vec, f)) return e;
  return cudaGetLastError();
}

// libjit_batchedadd_quantized (libjit.cpp:997-1015; entry points libjit_batchedadd_i8 and
// libjit_batchedadd_i32_i8, :1945-1969): a slice added to every slice of the batch.
template <typename SliceT>
__global__ void __launch_bounds__(kThreads) batched_add_i8_kernel(int8_t *__restrict__ dst, const int8_t *__restrict__ batch,
                                                                  const SliceT *__restrict__ slice, int64_t n,
                                                                  int64_t slice_size, int32_t dst_off, int32_t batch_off,
                                                                  int32_t slice_off, Triple bt, Triple st) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t b = (int32_t)batch[i] - batch_off;
    const int32_t sl = (int32_t)((uint32_t)(int32_t)slice[i % slice_size] - (uint32_t)slice_off);
    const int32_t x = scale32(b, bt.pre, bt.post, bt.scale, 0), y = scale32(sl, st.pre, st.post, st.scale, 0);
    dst[i] = (int8_t)clip_i8((int32_t)((uint32_t)x + (uint32_t)y + (uint32_t)dst_off));
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) splat_kernel(T *__restrict__ dst, int64_t n, T value) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = value;
}

// libjit_element_quantize_kernel_i8 (libjit.cpp:2997-3002): nearbyintf(x / scale + offset) in
// fp32 with round-half-even, then clip.  The division and the addition are separate roundings.
__device__ __forceinline__ int32_t quantize_one(float x, float scale, int32_t offset) {
  const float t = __fadd_rn(__fdiv_rn(x, scale), (float)offset);
  // values beyond the int32 range clip either way; keep the conversion defined
  const float c = fminf(fmaxf(nearbyintf(t), -2147483648.0f), 2147483520.0f);
  return clip_i8((int32_t)c);
}
// vec: both tensors 16-byte aligned -- four floats in, four bytes out per step
__global__ void __launch_bounds__(kThreads) quantize_i8_kernel(int8_t *__restrict__ dst, const float *__restrict__ src,
                                                               int64_t n, float scale, int32_t offset, int vec) {
  pdl_wait();
  pdl_launch_dependents();  // a contraction that follows may set up now (it waits for this kernel before its loads)
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t nv = vec ? (n >> 2) : 0;
  for (int64_t i = tid; i < nv; i += stride) {
    const float4 x = __ldg(reinterpret_cast<const float4 *>(src) + i);
    const uint32_t o = ((uint32_t)quantize_one(x.x, scale, offset) & 0xFFu) | (((uint32_t)quantize_one(x.y, scale, offset) & 0xFFu) << 8) |
                       (((uint32_t)quantize_one(x.z, scale, offset) & 0xFFu) << 16) | (((uint32_t)quantize_one(x.w, scale, offset) & 0xFFu) << 24);
    reinterpret_cast<uint32_t *>(dst)[i] = o;
  }
  for (int64_t i = (nv << 2) + tid; i < n; i += stride) dst[i] = (int8_t)quantize_one(src[i], scale, offset);
}

// libjit_element_dequantize_kernel_i8 (libjit.cpp:3014-3018)
__global__ void __launch_bounds__(kThreads) dequantize_i8_kernel(float *__restrict__ dst, const int8_t *__restrict__ src,
                                                                 int64_t n, float scale, int32_t offset, int vec) {
  pdl_wait();
  pdl_launch_dependents();  // a contraction that follows may set up now (it waits for this kernel before its loads)
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t nv = vec ? (n >> 2) : 0;
  for (int64_t i = tid; i < nv; i += stride) {
    const uint32_t q = __ldg(reinterpret_cast<const uint32_t *>(src) + i);
    float4 o;
    o.x = __fmul_rn(scale, (float)((int32_t)(int8_t)q - offset));
    o.y = __fmul_rn(scale, (float)((int32_t)(int8_t)(q >> 8) - offset));
    o.z = __fmul_rn(scale, (float)((int32_t)(int8_t)(q >> 16) - offset));
    o.w = __fmul_rn(scale, (float)((int32_t)(int8_t)(q >> 24) - offset));
    reinterpret_cast<float4 *>(dst)[i] = o;
  }
  for (int64_t i = (nv << 2) + tid; i < n; i += stride) dst[i] = __fmul_rn(scale, (float)((int32_t)src[i] - offset));
}

struct PoolGeom { int N, H, W, C, OH, OW, KH, KW, SH, SW, PT, PL; };

// libjit_max_pool_generic<int8_t> (libjit.cpp:811-870): cells outside the image are skipped,
// an empty window yields the default value (the output offset).
__global__ void __launch_bounds__(kThreads) max_pool_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out,
                                                               const __grid_constant__ PoolGeom g, int8_t def) {
  const int64_t total = (int64_t)g.N * g.OH * g.OW * g.C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.C);
    int64_t r = i / g.C;
    const int ow = (int)(r % g.OW);
    r /= g.OW;
    const int oh = (int)(r % g.OH), n = (int)(r / g.OH);
    int best = -129;
    for (int kh = 0; kh < g.KH; kh++)
      for (int kw = 0; kw < g.KW; kw++) {
        const int ih = oh * g.SH - g.PT + kh, iw = ow * g.SW - g.PL + kw;
        if (ih < 0 || iw < 0 || ih >= g.H || iw >= g.W) continue;
        const int v = in[(((int64_t)n * g.H + ih) * g.W + iw) * g.C + c];
        best = v > best ? v : best;
      }
    out[i] = best == -129 ? def : (int8_t)best;
  }
}

// The same for 16 channels per thread (C a multiple of 16, 16-byte aligned tensors): four
// byte-wise signed maxima per instruction.
__global__ void __launch_bounds__(kThreads) max_pool_i8_vec_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out,
                                                                   const __grid_constant__ PoolGeom g, int8_t def) {
  pdl_wait();
  pdl_launch_dependents();
  const int cc = g.C >> 4;
  const int64_t total = (int64_t)g.N * g.OH * g.OW * cc;
  const uint32_t lowest = 0x80808080u;  // four times -128
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % cc);
    int64_t r = i / cc;
    const int ow = (int)(r % g.OW);
    r /= g.OW;
    const int oh = (int)(r % g.OH), n = (int)(r / g.OH);
    uint4 best = make_uint4(lowest, lowest, lowest, lowest);
    bool any = false;
    for (int kh = 0; kh < g.KH; kh++)
      for (int kw = 0; kw < g.KW; kw++) {
        const int ih = oh * g.SH - g.PT + kh, iw = ow * g.SW - g.PL + kw;
        if (ih < 0 || iw < 0 || ih >= g.H || iw >= g.W) continue;
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(in + (((int64_t)n * g.H + ih) * g.W + iw) * g.C) + c);
        best.x = __vmaxs4(best.x, v.x);
        best.y = __vmaxs4(best.y, v.y);
        best.z = __vmaxs4(best.z, v.z);
        best.w = __vmaxs4(best.w, v.w);
        any = true;
      }
    if (!any) {
      const uint32_t d4 = 0x01010101u * (uint32_t)(uint8_t)def;
      best = make_uint4(d4, d4, d4, d4);
    }
    reinterpret_cast<uint4 *>(out)[i] = best;
  }
}

// libjit_avg_pool_i8 (libjit.cpp:2812-2897)
__global__ void __launch_bounds__(kThreads) avg_pool_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out,
                                                               const __grid_constant__ PoolGeom g, int count_include_pads,
                                                               int32_t out_off, int32_t in_off, Triple t) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t total = (int64_t)g.N * g.OH * g.OW * g.C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.C);
    int64_t r = i / g.C;
    const int ow = (int)(r % g.OW);
    r /= g.OW;
    const int oh = (int)(r % g.OH), n = (int)(r / g.OH);
    int32_t sum = 0, area = 0;
    const int ih0 = oh * g.SH - g.PT, iw0 = ow * g.SW - g.PL;
    if (ih0 >= 0 && iw0 >= 0 && ih0 + g.KH <= g.H && iw0 + g.KW <= g.W) {
      // the whole window is inside the image (a global average pool always): independent loads, four in
      // flight per thread -- a 7 x 7 window read one dependent byte at a time took 22 us for 131072 outputs
      const int8_t *p0 = in + (((int64_t)n * g.H + ih0) * g.W + iw0) * g.C + c;
      for (int kh = 0; kh < g.KH; kh++) {
        const int8_t *row = p0 + (int64_t)kh * g.W * g.C;
        int kw = 0;
        for (; kw + 4 <= g.KW; kw += 4) {
          const int32_t a0 = __ldg(row + (int64_t)kw * g.C), a1 = __ldg(row + (int64_t)(kw + 1) * g.C);
          const int32_t a2 = __ldg(row + (int64_t)(kw + 2) * g.C), a3 = __ldg(row + (int64_t)(kw + 3) * g.C);
          sum += (a0 + a1) + (a2 + a3);
        }
        for (; kw < g.KW; kw++) sum += __ldg(row + (int64_t)kw * g.C);
      }
      area = g.KH * g.KW;
      sum -= area * in_off;
    } else
    for (int kh = 0; kh < g.KH; kh++)
      for (int kw = 0; kw < g.KW; kw++) {
        const int ih = ih0 + kh, iw = iw0 + kw;
        if (ih < 0 || iw < 0 || ih >= g.H || iw >= g.W) continue;
        sum += (int32_t)in[(((int64_t)n * g.H + ih) * g.W + iw) * g.C + c] - in_off;
        area++;
      }
    int32_t res;
    if (count_include_pads) {
      res = clip_i8(scale32(sum, t.pre, t.post, t.scale, out_off));
    } else if (area == 0) {
      res = out_off;
    } else {
      // libjit_div_round_i32 (libjit_defs.h:238-244): round half away from zero
      const int32_t s = scale32(sum, t.pre, t.post, t.scale, 0);
      const int32_t rnd = area >> 1;
      res = clip_i8((s > 0 ? (s + rnd) / area : (s - rnd) / area) + out_off);
    }
    out[i] = (int8_t)res;
  }
}

// 4-D transpose by an arbitrary permutation (libjit_transpose_*, libjit.cpp:1945-...):
// dst dims = src dims permuted by `shuffle`; one thread per destination element.
// (F converts an element on its way: the identity, or the Quantize that a Transpose was sunk below.)
struct KeepF {
  template <typename T> __device__ __forceinline__ T operator()(T v) const { return v; }
};
struct QuantizeF {
  float scale;
  int32_t offset;
  __device__ __forceinline__ int8_t operator()(float v) const { return (int8_t)quantize_one(v, scale, offset); }
};
template <typename T, typename TO = T, typename F = KeepF>
__global__ void __launch_bounds__(kThreads) transpose4_kernel(const T *__restrict__ src, TO *__restrict__ dst, int d0, int d1,
                                                              int d2, int d3, int s0, int s1, int s2, int s3, F f = F()) {
  pdl_wait();
  pdl_launch_dependents();
  // d*: destination dims; s*: source element stride of each destination axis
  const int64_t total = (int64_t)d0 * d1 * d2 * d3;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int i3 = (int)(i % d3);
    int64_t r = i / d3;
    const int i2 = (int)(r % d2);
    r /= d2;
    const int i1 = (int)(r % d1), i0 = (int)(r / d1);
    dst[i] = f(src[(int64_t)i0 * s0 + (int64_t)i1 * s1 + (int64_t)i2 * s2 + (int64_t)i3 * s3]);
  }
}

// The same when the destination's innermost axis is short and its next axis is the source's innermost
// one (NCHW -> NHWC with few channels): one thread per destination "pixel" reads its d3 elements
// s3 apart -- neighbouring threads read neighbouring source elements -- and writes them side by side.
// (One thread per element read single bytes 50176 apart: 51 us for a 64 x 3 x 224 x 224 int8 tensor.)
template <typename T, typename TO = T, typename F = KeepF>
__global__ void __launch_bounds__(kThreads) transpose4_short_inner_kernel(const T *__restrict__ src, TO *__restrict__ dst, int d0,
                                                                          int d1, int d2, int d3, int s0, int s1, int s3,
                                                                          F f = F()) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t pixels = (int64_t)d0 * d1 * d2;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pixels; i += (int64_t)gridDim.x * blockDim.x) {
    const int i2 = (int)(i % d2);
    const int64_t r = i / d2;
    const int i1 = (int)(r % d1), i0 = (int)(r / d1);
    const T *from = src + (int64_t)i0 * s0 + (int64_t)i1 * s1 + i2;
    TO *to = dst + i * d3;
    for (int c = 0; c < d3; c++) to[c] = f(from[(int64_t)c * s3]);
  }
}

int pool_geom(PoolGeom &g, const int64_t *in_dims, const int64_t *out_dims, const int64_t *kernels, const int64_t *strides,
              const int64_t *pads) {
  GLOWB200_REQUIRE(in_dims && out_dims && kernels && strides && pads, "NULL shape array");
  for (int i = 0; i < 4; i++)
    GLOWB200_REQUIRE(in_dims[i] >= 0 && out_dims[i] >= 0 && in_dims[i] < (1ll << 31) && out_dims[i] < (1ll << 31),
                     "dimension out of range");
  GLOWB200_REQUIRE(in_dims[0] == out_dims[0] && in_dims[3] == out_dims[3], "pooling keeps batch and channels");
  GLOWB200_REQUIRE(kernels[0] >= 1 && kernels[1] >= 1 && strides[0] >= 1 && strides[1] >= 1, "bad kernel/stride");
  g.N = (int)in_dims[0]; g.H = (int)in_dims[1]; g.W = (int)in_dims[2]; g.C = (int)in_dims[3];
  g.OH = (int)out_dims[1]; g.OW = (int)out_dims[2];
  g.KH = (int)kernels[0]; g.KW = (int)kernels[1]; g.SH = (int)strides[0]; g.SW = (int)strides[1];
  g.PT = (int)pads[0]; g.PL = (int)pads[1];
  return GLOWB200_OK;
}

}  // namespace
}  // namespace glowb200

using namespace glowb200;

#define GLOWB200_STREAM reinterpret_cast<cudaStream_t>(stream)
#define GLOWB200_ELEMENTWISE_PROLOGUE(n, ...)                      \
  GLOWB200_REQUIRE((n) >= 0, "negative element count");            \
  if ((n) == 0) return GLOWB200_OK;                                \
  GLOWB200_REQUIRE(__VA_ARGS__, "NULL tensor pointer");

extern "C" int glowb200_element_add_i8(int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n, int32_t dest_offset,
                                       int32_t lhs_offset, int32_t rhs_offset, int32_t lhs_pre, int32_t lhs_post,
                                       int32_t lhs_scale, int32_t rhs_pre, int32_t rhs_post, int32_t rhs_scale,
                                       glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && lhs && rhs)
  GLOWB200_CUDA_OK(launch_map(dest, lhs, rhs, n,
                              AddF{dest_offset, lhs_offset, rhs_offset, Triple{lhs_pre, lhs_post, lhs_scale},
                                   Triple{rhs_pre, rhs_post, rhs_scale}, -128},
                              GLOWB200_STREAM));
  return GLOWB200_OK;
}

extern "C" int glowb200_element_binary_i8(int op, int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                                          int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset, int32_t lhs_pre,
                                          int32_t lhs_post, int32_t lhs_scale, int32_t rhs_pre, int32_t rhs_post,
                                          int32_t rhs_scale, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(op >= GLOWB200_BINARY_ADD && op <= GLOWB200_BINARY_MIN, "unknown binary operator %d", op);
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && lhs && rhs)
  const Triple lt{lhs_pre, lhs_post, lhs_scale}, rt{rhs_pre, rhs_post, rhs_scale};
  cudaError_t e;
  switch (op) {
    case GLOWB200_BINARY_ADD:
      e = launch_map(dest, lhs, rhs, n, AddF{dest_offset, lhs_offset, rhs_offset, lt, rt, -128}, GLOWB200_STREAM);
      break;
    case GLOWB200_BINARY_SUB:
      e = launch_map(dest, lhs, rhs, n, BinaryF<1>{dest_offset, lhs_offset, rhs_offset, lt, rt}, GLOWB200_STREAM);
      break;
    case GLOWB200_BINARY_MAX:
      e = launch_map(dest, lhs, rhs, n, BinaryF<2>{dest_offset, lhs_offset, rhs_offset, lt, rt}, GLOWB200_STREAM);
      break;
    default:
      e = launch_map(dest, lhs, rhs, n, BinaryF<3>{dest_offset, lhs_offset, rhs_offset, lt, rt}, GLOWB200_STREAM);
      break;
  }
  GLOWB200_CUDA_OK(e);
  return GLOWB200_OK;
}

extern "C" int glowb200_element_muldiv_i8(int is_div, int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                                          int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset, int32_t pre,
                                          int32_t post, int32_t scale, glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && lhs && rhs)
  if (is_div)
    GLOWB200_CUDA_OK(launch_map(dest, lhs, rhs, n, MulDivF<true>{dest_offset, lhs_offset, rhs_offset, Triple{pre, post, scale}},
                                GLOWB200_STREAM));
  else
    GLOWB200_CUDA_OK(launch_map(dest, lhs, rhs, n, MulDivF<false>{dest_offset, lhs_offset, rhs_offset, Triple{pre, post, scale}},
                                GLOWB200_STREAM));
  return GLOWB200_OK;
}

extern "C" int glowb200_batched_add_i8(int8_t *dest, const int8_t *batch, const void *slice, int slice_is_int32,
                                       int64_t num_slices, int64_t slice_size, int32_t dest_offset, int32_t batch_offset,
                                       int32_t slice_offset, int32_t batch_pre, int32_t batch_post, int32_t batch_scale,
                                       int32_t slice_pre, int32_t slice_post, int32_t slice_scale, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(num_slices >= 0 && slice_size >= 0 && num_slices < (1ll << 31) && slice_size < (1ll << 31),
                   "bad slice count / size");
  const int64_t n = num_slices * slice_size;
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && batch && slice)
  const Triple bt{batch_pre, batch_post, batch_scale}, st{slice_pre, slice_post, slice_scale};
  if (slice_is_int32)
    batched_add_i8_kernel<int32_t><<<grid_for(n), kThreads, 0, GLOWB200_STREAM>>>(
        dest, batch, reinterpret_cast<const int32_t *>(slice), n, slice_size, dest_offset, batch_offset, slice_offset, bt, st);
  else
    batched_add_i8_kernel<int8_t><<<grid_for(n), kThreads, 0, GLOWB200_STREAM>>>(
        dest, batch, reinterpret_cast<const int8_t *>(slice), n, slice_size, dest_offset, batch_offset, slice_offset, bt, st);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

extern "C" int glowb200_element_add_maxsplat_i8(int8_t *dest, const int8_t *lhs, const int8_t *rhs, int64_t n,
                                                int32_t dest_offset, int32_t lhs_offset, int32_t rhs_offset, int32_t lhs_pre,
                                                int32_t lhs_post, int32_t lhs_scale, int32_t rhs_pre, int32_t rhs_post,
                                                int32_t rhs_scale, int32_t splat, glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && lhs && rhs)
  GLOWB200_REQUIRE(splat >= -128 && splat <= 127, "splat value outside int8");
  GLOWB200_CUDA_OK(launch_map(dest, lhs, rhs, n,
                              AddF{dest_offset, lhs_offset, rhs_offset, Triple{lhs_pre, lhs_post, lhs_scale},
                                   Triple{rhs_pre, rhs_post, rhs_scale}, splat},
                              GLOWB200_STREAM));
  return GLOWB200_OK;
}

extern "C" int glowb200_element_relu_i8(int8_t *dest, const int8_t *src, int64_t n, int32_t src_offset, int32_t dest_offset,
                                        int32_t dest_pre, int32_t dest_post, int32_t dest_scale, glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && src)
  GLOWB200_CUDA_OK(launch_map(dest, src, nullptr, n, ReluF{src_offset, dest_offset, Triple{dest_pre, dest_post, dest_scale}},
                              GLOWB200_STREAM));
  return GLOWB200_OK;
}

extern "C" int glowb200_element_maxsplat_i8(int8_t *dest, const int8_t *src, int64_t n, int32_t splat,
                                            glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && src)
  GLOWB200_REQUIRE(splat >= -128 && splat <= 127, "splat value outside int8");
  GLOWB200_CUDA_OK(launch_map(dest, src, nullptr, n, MaxSplatF{splat}, GLOWB200_STREAM));
  return GLOWB200_OK;
}

extern "C" int glowb200_splat_f(void *dest, int64_t n, float value, int dest_is_fp16, glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest)
  if (dest_is_fp16) splat_kernel<__half><<<grid_for(n), kThreads, 0, GLOWB200_STREAM>>>(reinterpret_cast<__half *>(dest), n, __float2half_rn(value));
  else splat_kernel<float><<<grid_for(n), kThreads, 0, GLOWB200_STREAM>>>(reinterpret_cast<float *>(dest), n, value);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

extern "C" int glowb200_element_rescale_i8(int8_t *dest, const int8_t *src, int64_t n, int32_t out_offset, int32_t in_offset,
                                           int32_t pre, int32_t post, int32_t scale, glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && src)
  GLOWB200_CUDA_OK(launch_map(dest, src, nullptr, n, RescaleF{out_offset, in_offset, Triple{pre, post, scale}}, GLOWB200_STREAM));
  return GLOWB200_OK;
}

extern "C" int glowb200_element_quantize_i8(int8_t *dest, const float *src, int64_t n, float scale, int32_t offset,
                                            glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && src)
  const int vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dest) & 3u) == 0;
  GLOWB200_CUDA_OK(launch_pdl(quantize_i8_kernel, grid_for(vec ? (n + 3) / 4 : n), kThreads, 0, GLOWB200_STREAM, dest, src, n, scale, offset, vec));
  return GLOWB200_OK;
}

extern "C" int glowb200_element_dequantize_i8(float *dest, const int8_t *src, int64_t n, float scale, int32_t offset,
                                              glowb200_stream_t stream) {
  GLOWB200_ELEMENTWISE_PROLOGUE(n, dest && src)
  const int vec = (reinterpret_cast<uintptr_t>(dest) & 15u) == 0 && (reinterpret_cast<uintptr_t>(src) & 3u) == 0;
  GLOWB200_CUDA_OK(launch_pdl(dequantize_i8_kernel, grid_for(vec ? (n + 3) / 4 : n), kThreads, 0, GLOWB200_STREAM, dest, src, n, scale, offset, vec));
  return GLOWB200_OK;
}

extern "C" int glowb200_max_pool_i8(const int8_t *in, int8_t *out, const int64_t *in_dims, const int64_t *out_dims,
                                    const int64_t *kernels, const int64_t *strides, const int64_t *pads, int32_t out_offset,
                                    glowb200_stream_t stream) {
  PoolGeom g;
  if (int rc = pool_geom(g, in_dims, out_dims, kernels, strides, pads)) return rc;
  const int64_t total = (int64_t)g.N * g.OH * g.OW * g.C;
  if (total == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(in && out, "NULL tensor pointer");
  if ((g.C & 15) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0)
    GLOWB200_CUDA_OK(launch_pdl(max_pool_i8_vec_kernel, grid_for(total >> 4), kThreads, 0, GLOWB200_STREAM, in, out, g, (int8_t)out_offset));
  else
    max_pool_i8_kernel<<<grid_for(total), kThreads, 0, GLOWB200_STREAM>>>(in, out, g, (int8_t)out_offset);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

extern "C" int glowb200_avg_pool_i8(const int8_t *in, int8_t *out, const int64_t *in_dims, const int64_t *out_dims,
                                    const int64_t *kernels, const int64_t *strides, const int64_t *pads,
                                    int count_include_pads, int32_t out_offset, int32_t in_offset, int32_t out_pre,
                                    int32_t out_post, int32_t out_scale, glowb200_stream_t stream) {
  PoolGeom g;
  if (int rc = pool_geom(g, in_dims, out_dims, kernels, strides, pads)) return rc;
  const int64_t total = (int64_t)g.N * g.OH * g.OW * g.C;
  if (total == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(in && out, "NULL tensor pointer");
  GLOWB200_CUDA_OK(launch_pdl(avg_pool_i8_kernel, grid_for(total), kThreads, 0, GLOWB200_STREAM, in, out, g, count_include_pads ? 1 : 0,
                              out_offset, in_offset, Triple{out_pre, out_post, out_scale}));
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}

namespace {
// Destination dims d[] and, per destination axis, the source's element stride st[] of a shuffle of up to 4 axes.
struct TransposePlan { int d[4], st[4]; int64_t total; };
int plan_transpose(TransposePlan &t, const int64_t *src_dims, const int32_t *shuffle, int num_dims) {
  GLOWB200_REQUIRE(src_dims && shuffle && num_dims >= 1 && num_dims <= 4, "1 to 4 dimensions are supported");
  int64_t sd[4] = {1, 1, 1, 1}, sstride[4];
  int sh[4] = {0, 1, 2, 3};
  const int lead = 4 - num_dims;  // pad with leading unit axes
  bool seen[4] = {false, false, false, false};
  for (int i = 0; i < num_dims; i++) {
    GLOWB200_REQUIRE(src_dims[i] >= 0 && src_dims[i] < (1ll << 31), "dimension out of range");
    GLOWB200_REQUIRE(shuffle[i] >= 0 && shuffle[i] < num_dims && !seen[shuffle[i]], "shuffle is not a permutation");
    seen[shuffle[i]] = true;
    sd[lead + i] = src_dims[i];
    sh[lead + i] = lead + shuffle[i];
  }
  sstride[3] = 1;
  for (int i = 2; i >= 0; i--) sstride[i] = sstride[i + 1] * sd[i + 1];
  t.total = sd[0] * sd[1] * sd[2] * sd[3];
  GLOWB200_REQUIRE(t.total < (1ll << 31), "tensor too large for this kernel");
  for (int i = 0; i < 4; i++) {
    t.d[i] = (int)sd[sh[i]];
    t.st[i] = (int)sstride[sh[i]];
  }
  return GLOWB200_OK;
}

template <typename T, typename TO, typename F>
int run_transpose(const TransposePlan &t, const T *src, TO *dest, F f, cudaStream_t s) {
  if (t.d[3] <= 16 && t.st[2] == 1 && t.st[3] != 1)
    GLOWB200_CUDA_OK(launch_pdl(transpose4_short_inner_kernel<T, TO, F>, grid_for(t.total / t.d[3]), kThreads, 0, s, src, dest, t.d[0],
                                t.d[1], t.d[2], t.d[3], t.st[0], t.st[1], t.st[3], f));
  else
    GLOWB200_CUDA_OK(launch_pdl(transpose4_kernel<T, TO, F>, grid_for(t.total), kThreads, 0, s, src, dest, t.d[0], t.d[1], t.d[2], t.d[3],
                                t.st[0], t.st[1], t.st[2], t.st[3], f));
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}
}  // namespace

extern "C" int glowb200_transpose(const void *src, void *dest, const int64_t *src_dims, const int32_t *shuffle, int num_dims,
                                  int element_bytes, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(element_bytes == 1 || element_bytes == 4, "element size must be 1 or 4 bytes");
  TransposePlan t;
  if (int rc = plan_transpose(t, src_dims, shuffle, num_dims)) return rc;
  if (t.total == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(src && dest, "NULL tensor pointer");
  if (element_bytes == 1)
    return run_transpose(t, reinterpret_cast<const int8_t *>(src), reinterpret_cast<int8_t *>(dest), KeepF(), GLOWB200_STREAM);
  return run_transpose(t, reinterpret_cast<const float *>(src), reinterpret_cast<float *>(dest), KeepF(), GLOWB200_STREAM);
}

extern "C" int glowb200_quantize_transpose_i8(int8_t *dest, const float *src, const int64_t *src_dims, const int32_t *shuffle,
                                              int num_dims, float scale, int32_t offset, glowb200_stream_t stream) {
  TransposePlan t;
  if (int rc = plan_transpose(t, src_dims, shuffle, num_dims)) return rc;
  if (t.total == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(src && dest, "NULL tensor pointer");
  GLOWB200_REQUIRE(scale != 0.0f, "scale must not be zero");
  return run_transpose(t, src, dest, QuantizeF{scale, offset}, GLOWB200_STREAM);
}
