// Symmetric (peer-mapped) memory on one NVLink/NVSwitch node.
//
// Each rank allocates its exchange buffers with cudaMalloc, exports a CUDA IPC handle, and maps
// every peer's buffer into its own address space; kernels then read and write peer memory with
// plain ld/st over NVLink. Handles travel through the process group's object collective on the
// Python side (pithtrain_b200/parallel/symm_mem.py). The reference has no counterpart: all of its
// inter-GPU traffic goes through NCCL (pithtrain/modules/distributed.py:96-97).
#include <string.h>

#include "host_common.h"

PT_API int pt_symm_malloc(void** out, long long bytes) {
  if (!out || bytes <= 0) return -1;
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(*out, 0, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaDeviceSynchronize();
}

PT_API int pt_symm_free(void* p) { return (int)cudaFree(p); }

// handle: 64 bytes (cudaIpcMemHandle_t)
PT_API int pt_ipc_export(void* p, unsigned char* handle) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle, &h, sizeof(h));
  return 0;
}

PT_API int pt_ipc_import(const unsigned char* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}

PT_API int pt_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

PT_API int pt_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

// 1 when `dev` can map memory of `peer` (same node, NVLink or PCIe P2P).
PT_API int pt_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}
