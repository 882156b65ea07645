// Buffers that the other GPUs of the node can write into: the receive side of the pooled-
// embedding exchange.  One process per GPU; a buffer is plain device memory exported with a
// CUDA IPC handle (64 opaque bytes that the host side passes between the processes), mapped
// by each peer with lazily enabled peer access.  Kernels then store to it with ordinary
// stores over NVLink -- no multicast object is ever created or bound.
//
// These four calls are set-up / tear-down API: create and destroy allocate and free device
// memory and belong at network-load time, never on the request path.
#include <cstring>

#include "common.cuh"

extern "C" int glowb200_peer_buffer_create(size_t bytes, void **device_ptr, void *ipc_handle_64_bytes) {
  GLOWB200_REQUIRE(bytes > 0 && device_ptr && ipc_handle_64_bytes, "bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void *p = nullptr;
  GLOWB200_CUDA_OK(cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return glowb200::set_error(GLOWB200_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  memcpy(ipc_handle_64_bytes, &h, 64);
  *device_ptr = p;
  return GLOWB200_OK;
}

extern "C" int glowb200_peer_buffer_open(const void *ipc_handle_64_bytes, void **device_ptr) {
  GLOWB200_REQUIRE(ipc_handle_64_bytes && device_ptr, "bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle_64_bytes, 64);
  GLOWB200_CUDA_OK(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return GLOWB200_OK;
}

extern "C" int glowb200_peer_buffer_close(void *device_ptr) {
  if (device_ptr) GLOWB200_CUDA_OK(cudaIpcCloseMemHandle(device_ptr));
  return GLOWB200_OK;
}

extern "C" int glowb200_peer_buffer_destroy(void *device_ptr) {
  if (device_ptr) GLOWB200_CUDA_OK(cudaFree(device_ptr));
  return GLOWB200_OK;
}

// ------------------------------------------------------------------------------------------
// Rendezvous of the ranks that store into each other's buffers: "every rank's stores of this
// step are complete" without a collective library call.
//
// Every rank owns a small flag buffer (glowb200_peer_buffer_create, 8 * (world + 1) bytes, zeroed)
// that its peers have mapped: slot r is written by rank r, slot `world` is the rank's own count
// of the rendezvous it has made.  One launch of one warp per rendezvous: lane r tells peer r
// "my step e is stored" (a system-scope release store into slot `rank` of r's buffer, behind a
// system-scope fence that orders the kernel's predecessors' stores -- the pooling kernel that
// ran before it on the stream -- ahead of the flag), then waits until its own slot r reads e or
// more (acquire loads).  The step count e lives in the rank's own buffer and is advanced by the
// kernel itself, so the launch can be replayed from a CUDA graph.  The wait is bounded: after
// `limit_cycles` SM clocks it raises GLOWB200_STATUS_WAIT_TIMEOUT and the kernel returns.
// Ordinary peer loads and stores only.
// ------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(32) peer_rendezvous_kernel(unsigned long long *mine, unsigned long long *const *peers,
                                                             int world, int rank, long long limit_cycles, int32_t *status) {
  const int lane = threadIdx.x;
  unsigned long long e = 0;
  if (lane == 0) {
    e = mine[world] + 1;
    mine[world] = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  __threadfence_system();
  if (lane < world) {
    unsigned long long *slot = peers[lane] + rank;  // slot `rank` of peer `lane` (of this rank's own buffer for lane == rank)
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(slot), "l"(e) : "memory");
    const long long t0 = clock64();
    bool ok = false;
    while (true) {
      unsigned long long seen;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(mine + lane) : "memory");
      if (seen >= e) { ok = true; break; }
      if (clock64() - t0 > limit_cycles) break;
    }
    if (!ok && status != nullptr) atomicOr(status, GLOWB200_STATUS_WAIT_TIMEOUT);
  }
}
}  // namespace

extern "C" int glowb200_peer_rendezvous(void *my_flags, void *const *peer_flags_device_array, int world, int rank,
                                        int64_t limit_cycles, int32_t *status, glowb200_stream_t stream) {
  GLOWB200_REQUIRE(my_flags && peer_flags_device_array && world >= 1 && world <= 32 && rank >= 0 && rank < world && limit_cycles > 0,
                   "bad arguments (at most 32 ranks)");
  peer_rendezvous_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<unsigned long long *>(my_flags), reinterpret_cast<unsigned long long *const *>(peer_flags_device_array), world,
      rank, (long long)limit_cycles, status);
  GLOWB200_CUDA_OK(cudaGetLastError());
  return GLOWB200_OK;
}
