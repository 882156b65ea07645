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
