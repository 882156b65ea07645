// Quantization profiling on the device: the running min / max and histogram of a tensor.
//
// Reference: libjit_quantization_profile (lib/LLVMIRCodeGen/libjit/libjit.cpp:3440-3523), itself a
// port of generateTensorHistogram (lib/Quantization/Base/Profile.cpp:36-112): the node Glow
// inserts behind every value while it profiles a network for quantization.  Off the inference
// path; here so that profiling a model whose activations already live on the GPU does not pull
// them to the host.
//
// Three launches: (1) min / max of the input (grid-wide reduction through a partials array);
// (2) one thread merges them into the running range and, when the range grew, redistributes the
// existing bins exactly as the reference's sequential loop does; (3) the bin of every element is
// counted in shared memory (exact integers), and the counts are added to the float histogram the
// way repeated `+= 1.0f` would: exact up to 2^24, where a float stops counting.
#include "common.cuh"

namespace glowb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxBlocks = 1184;   // 8 per SM
constexpr int kSharedBins = 8192;  // 32 KB of counters

// get_bin (libjit.cpp:1046-1052)
__device__ __forceinline__ unsigned long long get_bin(unsigned long long bins, float width, float minv, float v) {
  if (width == 0.0f) return 0;
  const unsigned long long b = (unsigned long long)__fdiv_rn(__fsub_rn(v, minv), width);
  return b < bins - 1 ? b : bins - 1;
}

__global__ void __launch_bounds__(kThreads) min_max_kernel(const float *__restrict__ x, long long n, float *partials) {
  __shared__ float s_mn[kThreads / 32], s_mx[kThreads / 32];
  float mn = x[0], mx = mn;
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads) {
    const float v = x[i];
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
    for (int i = 1; i < kThreads / 32; i++) {
      mn = s_mn[i] < mn ? s_mn[i] : mn;
      mx = s_mx[i] > mx ? s_mx[i] : mx;
    }
    partials[2 * blockIdx.x] = mn;
    partials[2 * blockIdx.x + 1] = mx;
  }
}

// One thread: the scalar part of the reference, kept in its order.  range[0..1] receive the
// (min, max) the new elements are binned with.
__global__ void merge_range_kernel(const float *partials, int blocks, float *comp_info, float *hist, long long bins,
                                   float *scaled, float *range) {
  float min_in = partials[0], max_in = partials[1];
  for (int i = 1; i < blocks; i++) {
    min_in = partials[2 * i] < min_in ? partials[2 * i] : min_in;
    max_in = partials[2 * i + 1] > max_in ? partials[2 * i + 1] : max_in;
  }
  float mn = comp_info[0], mx = comp_info[1];
  const float new_min = min_in < mn ? min_in : mn, new_max = max_in > mx ? max_in : mx;
  comp_info[0] = new_min;
  comp_info[1] = new_max;
  if (bins == 0) return;
  bool all_zero = true;
  for (long long i = 0; i < bins && all_zero; i++) all_zero = hist[i] == 0.0f;
  if (all_zero) {
    mn = min_in;
    mx = max_in;
  }
  if (new_min < mn || new_max > mx) {
    const float fbins = (float)(unsigned long long)bins;
    const float dest_w = __fdiv_rn(__fsub_rn(new_max, new_min), fbins), src_w = __fdiv_rn(__fsub_rn(mx, mn), fbins);
    for (long long i = 0; i < bins; i++) scaled[i] = 0.0f;
    for (long long i = 0; i < bins; i++) {
      const float h = hist[i];
      if (h == 0.0f) continue;
      const float src_begin = __fadd_rn(mn, __fmul_rn(src_w, (float)(unsigned long long)i));
      const unsigned long long dest_bin = (unsigned long long)__fdiv_rn(__fsub_rn(src_begin, new_min), dest_w);
      const float dest_end = __fadd_rn(new_min, __fmul_rn(dest_w, (float)(dest_bin + 1)));
      const float share = __fmul_rn(__fdiv_rn(__fsub_rn(dest_end, src_begin), src_w), h);
      const float rounded = (float)round((double)share);
      const unsigned long long cnt = (unsigned long long)(rounded < h ? rounded : h);
      unsigned long long nb = get_bin((unsigned long long)bins, dest_w, new_min, src_begin);
      scaled[nb] = __fadd_rn(scaled[nb], (float)cnt);
      if ((float)cnt < h) {
        nb = get_bin((unsigned long long)bins, dest_w, new_min, __fadd_rn(src_begin, dest_w));
        scaled[nb] = __fadd_rn(scaled[nb], __fsub_rn(h, (float)cnt));
      }
    }
    for (long long i = 0; i < bins; i++) hist[i] = scaled[i];
    mn = new_min;
    mx = new_max;
  }
  range[0] = mn;
  range[1] = mx;
}

// counts[b] += number of elements that fall into bin b (shared-memory counters when the bins fit).
__global__ void __launch_bounds__(kThreads) count_bins_kernel(const float *__restrict__ x, long long n, const float *range,
                                                              long long bins, unsigned long long *counts) {
  __shared__ unsigned int s_counts[kSharedBins];
  const bool shared = bins <= kSharedBins;
  if (shared)
    for (int i = threadIdx.x; i < bins; i += kThreads) s_counts[i] = 0;
  __syncthreads();
  const float mn = range[0];
  const float width = __fdiv_rn(__fsub_rn(range[1], mn), (float)(unsigned long long)bins);
  for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kThreads) {
    const unsigned long long b = get_bin((unsigned long long)bins, width, mn, x[i]);
    if (shared) atomicAdd(&s_counts[b], 1u);
    else atomicAdd(&counts[b], 1ull);
  }
  __syncthreads();
  if (shared)
    for (int i = threadIdx.x; i < bins; i += kThreads)
      if (s_counts[i]) atomicAdd(&counts[i], (unsigned long long)s_counts[i]);
}

// hist[b] after `counts[b]` increments by 1.0f: a float counts exactly up to 2^24 and then stays.
__global__ void __launch_bounds__(kThreads) add_counts_kernel(float *hist, const unsigned long long *counts, long long bins) {
  const long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
  if (i >= bins) return;
  const unsigned long long c = counts[i];
  if (c == 0) return;
  const float h = hist[i];
  // the increments are exact while the value is an integer below 2^24 (it always is an integer:
  // counts and redistributed counts); anything else falls back to adding one by one
  if (h >= 0.0f && h <= 16777216.0f && h == truncf(h)) {
    const unsigned long long total = (unsigned long long)h + c;
    hist[i] = total <= 16777216ull ? (float)total : 16777216.0f;
  } else {
    float v = h;
    for (unsigned long long k = 0; k < c; k++) {
      const float nv = __fadd_rn(v, 1.0f);
      if (nv == v) break;
      v = nv;
    }
    hist[i] = v;
  }
}

}  // namespace
}  // namespace glowb200

using namespace glowb200;

extern "C" size_t glowb200_quantization_profile_workspace_bytes(int64_t bins) {
  if (bins < 0) return 0;
  return align_up((size_t)kMaxBlocks * 8, 256) + 256 + align_up((size_t)bins * 4, 256) + align_up((size_t)bins * 8, 256);
}

extern "C" int glowb200_quantization_profile(const float *input, int64_t size, float *comp_info, float *histogram,
                                             int64_t bins, void *workspace, size_t workspace_bytes,
                                             glowb200_stream_t stream) {
  GLOWB200_REQUIRE(size > 0 && bins >= 0 && bins < (1ll << 31), "size must be positive, bins in [0, 2^31)");
  GLOWB200_REQUIRE(input != nullptr && comp_info != nullptr && (bins == 0 || histogram != nullptr), "NULL tensor pointer");
  const size_t need = glowb200_quantization_profile_workspace_bytes(bins);
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(GLOWB200_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  GLOWB200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 7) == 0, "workspace must be 8-byte aligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  uint8_t *w = reinterpret_cast<uint8_t *>(workspace);
  float *partials = reinterpret_cast<float *>(w);
  w += align_up((size_t)kMaxBlocks * 8, 256);
  float *range = reinterpret_cast<float *>(w);
  w += 256;
  float *scaled = reinterpret_cast<float *>(w);
  w += align_up((size_t)bins * 4, 256);
  unsigned long long *counts = reinterpret_cast<unsigned long long *>(w);
  int blocks = (int)((size + kThreads - 1) / kThreads);
  blocks = blocks > kMaxBlocks ? kMaxBlocks : blocks;
  min_max_kernel<<<blocks, kThreads, 0, s>>>(input, size, partials);
  GLOWB200_CUDA_OK(cudaGetLastError());
  merge_range_kernel<<<1, 1, 0, s>>>(partials, blocks, comp_info, histogram, bins, scaled, range);
  GLOWB200_CUDA_OK(cudaGetLastError());
  if (bins == 0) return GLOWB200_OK;
  GLOWB200_CUDA_OK(cudaMemsetAsync(counts, 0, (size_t)bins * 8, s));
  count_bins_kernel<<<blocks, kThreads, 0, s>>>(input, size, range, bins, counts);
  GLOWB200_CUDA_OK(cudaGetLastError());
  add_counts_kernel<<<(unsigned)((bins + kThreads - 1) / kThreads), kThreads, 0, s>>>(histogram, counts, bins);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}
