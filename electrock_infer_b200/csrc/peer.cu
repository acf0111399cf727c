// Peer-visible device buffers for the expert-parallel layer: plain cudaMalloc allocations shared
// between the rank processes of one node with CUDA IPC handles (no multicast objects are
// created).  These are set-up calls: they allocate, synchronise and are not for the hot path.
#include <string.h>

#include "common.cuh"

extern "C" int b200moe_peer_alloc(size_t bytes, void** ptr, void* ipc_handle_64) {
  using namespace b200moe;
  if (!ptr || !ipc_handle_64 || bytes == 0) return fail(B200MOE_ERR_NULL, "peer_alloc: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "peer_alloc: cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(ipc_handle_64), p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(B200MOE_ERR_CUDA, "peer_alloc: %s", cudaGetErrorString(e));
  }
  *ptr = p;
  return B200MOE_OK;
}

extern "C" int b200moe_peer_open(const void* ipc_handle_64, void** ptr) {
  using namespace b200moe;
  if (!ptr || !ipc_handle_64) return fail(B200MOE_ERR_NULL, "peer_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle_64, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "peer_open: %s", cudaGetErrorString(e));
  *ptr = p;
  return B200MOE_OK;
}

extern "C" int b200moe_peer_close(void* ptr) {
  using namespace b200moe;
  if (!ptr) return B200MOE_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "peer_close: %s", cudaGetErrorString(e));
  return B200MOE_OK;
}

extern "C" int b200moe_peer_free(void* ptr) {
  using namespace b200moe;
  if (!ptr) return B200MOE_OK;
  const cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "peer_free: %s", cudaGetErrorString(e));
  return B200MOE_OK;
}
