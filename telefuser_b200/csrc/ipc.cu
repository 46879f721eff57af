// Peer-mapped ("symmetric") buffers for the ranks of one node: each rank allocates a buffer, publishes
// its CUDA IPC handle, and maps every other rank's buffer. The mappings are plain device pointers
// usable by any kernel (peer loads / stores over NVLink).
// The reference has no counterpart: its ranks exchange data only through NCCL (telefuser/distributed/).
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "tfb_api.h"
#include "tfb_common.cuh"

using namespace tfb;

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");

extern "C" int tfb_ipc_alloc(long bytes, void** ptr, void* handle64) {
  if (bytes <= 0 || !ptr || !handle64) return TFB_ERR_BAD_SHAPE;
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) return TFB_ERR_TOO_LARGE;
  if (cudaMemset(p, 0, static_cast<size_t>(bytes)) != cudaSuccess) {
    cudaFree(p);
    return TFB_ERR_LAUNCH;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return TFB_ERR_NO_DRIVER;
  }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return TFB_OK;
}

extern "C" int tfb_ipc_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return TFB_ERR_BAD_SHAPE;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return TFB_ERR_NO_DRIVER;
  }
  *ptr = p;
  return TFB_OK;
}

extern "C" int tfb_ipc_close(void* ptr) {
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}

extern "C" int tfb_ipc_free(void* ptr) {
  return cudaFree(ptr) == cudaSuccess ? TFB_OK : TFB_ERR_LAUNCH;
}
