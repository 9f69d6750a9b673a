// Peer-mapped device buffers through CUDA IPC (one process per GPU, same node).
// A buffer is a plain cudaMalloc allocation, zero-filled; its IPC handle is exchanged by the
// caller (e.g. through torch.distributed) and opened in the peers, which also turns on peer
// access over NVLink.  Kernels then read and write it with ordinary loads and stores.
#include <string.h>

#include "common.cuh"

using namespace tp;

extern "C" void* tp_symm_alloc(long long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) return nullptr;
  if (cudaMemset(p, 0, static_cast<size_t>(bytes)) != cudaSuccess) {
    cudaFree(p);
    return nullptr;
  }
  cudaDeviceSynchronize();
  return p;
}

extern "C" int tp_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? kOk : kErrDriver; }

// handle: 64 bytes
extern "C" int tp_ipc_export(void* p, unsigned char* handle) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return kErrDriver;
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(handle, &h, sizeof(h));
  return kOk;
}

extern "C" void* tp_ipc_import(const unsigned char* handle) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

extern "C" int tp_ipc_close(void* p) {
  return cudaIpcCloseMemHandle(p) == cudaSuccess ? kOk : kErrDriver;
}
