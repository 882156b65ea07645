// Shared host/device helpers of the glow_b200 kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "glow_b200.h"

namespace glowb200 {

// Thread-local message behind glowb200_last_error().
char *last_error_buffer();
int set_error(int code, const char *fmt, ...);

#define GLOWB200_CUDA_OK(expr)                                                                  \
  do {                                                                                          \
    cudaError_t e__ = (expr);                                                                   \
    if (e__ != cudaSuccess)                                                                     \
      return ::glowb200::set_error(GLOWB200_ERR_CUDA, "%s failed: %s", #expr,                   \
                                   cudaGetErrorString(e__));                                    \
  } while (0)

#define GLOWB200_REQUIRE(cond, ...)                                                             \
  do {                                                                                          \
    if (!(cond)) return ::glowb200::set_error(GLOWB200_ERR_INVALID_ARGUMENT, __VA_ARGS__);      \
  } while (0)

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Number of SMs of the current device (cached per device).
int sm_count();

// Bag boundaries of one lengths array (defined beside the gather-pool kernels):
// seg_begin[i] = min(sum(max(lengths[0..i), 0)), num_indices) for i in [0, segments]; the array
// must hold glowb200_slws_workspace_bytes(segments, 1) bytes.  Raises the status bits of
// negative lengths and of lengths that overrun num_indices.
int launch_segments_from_lengths(const int32_t *lengths, int64_t segments, int64_t num_indices,
                                 void *workspace, size_t workspace_bytes, int32_t *status,
                                 cudaStream_t stream);

// ---- integer requantisation (device side) ----------------------------------------------
// libjit_scale<int32,int32> (lib/LLVMIRCodeGen/libjit/libjit_defs.h:158-173): arithmetic
// shifts, 32-bit wrapping multiply/add, rounding term only when post > 0, offset added last.
__host__ __device__ __forceinline__ int32_t scale32(int32_t input, int32_t pre, int32_t post,
                                                    int32_t scale, int32_t offset) {
  const uint32_t rtn = (post > 0) ? (1u << (post - 1)) : 0u;
  const int32_t a = input >> pre;
  const int32_t c = (int32_t)((uint32_t)a * (uint32_t)scale + rtn);
  return (int32_t)((uint32_t)(c >> post) + (uint32_t)offset);
}

// libjit_clip_i8 (libjit_defs.h:146-148).
__host__ __device__ __forceinline__ int32_t clip_i8(int32_t v) {
  return v < -128 ? -128 : (v > 127 ? 127 : v);
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start (set up its barriers, tensor memory, shared memory) while the kernel before it in the stream
// is still running, once every block of that kernel has passed pdl_launch_dependents(); it must not
// touch global memory before pdl_wait(), which returns when the earlier kernel has completed and its
// writes are visible.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Programmatic launches are on unless the environment says GLOWB200_PDL=0 (read once).  A waiting
// kernel holds its shared memory and thread slots, which costs a kernel that runs beside it on
// another stream: a caller that overlaps streams can switch them off.
bool pdl_enabled();
// Launches `kernel` so that it may start beside the tail of the kernel before it (see pdl_wait()).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, unsigned block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace glowb200
