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

// ----------------------------------------------------------------------------------------------
// Building blocks for protocols over symmetric memory: system-scope flag words and bulk copies
// whose source or destination may be a peer mapping. Every wait is bounded and reports through the
// library's status word (code PT_ERR_TIMEOUT_PEER).
// ----------------------------------------------------------------------------------------------
#include "ptx.cuh"
#include "peer_wait.cuh"

namespace pt {
namespace symm {

constexpr int MAXW = 32;
struct PtrList {
  unsigned* p[MAXW];
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// word `index` of every listed control block = value, ordered after all earlier work of the stream
__global__ void signal_kernel(PtrList ctl, int n, int index, unsigned value) {
  __threadfence_system();
  if ((int)threadIdx.x < n) st_release_sys(ctl.p[threadIdx.x] + index, value);
}

// wait until words [index, index + count) of the local control block are >= value (wrap-safe)
__global__ void wait_kernel(const unsigned* ctl, int index, int count, unsigned value, int* err) {
  if ((int)threadIdx.x >= count) return;
  const unsigned* p = ctl + index + threadIdx.x;
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if ((int)(ld_acquire_sys(p) - value) >= 0) return;
    if ((it & 255u) == 255u) {
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > pt_peer_wait_limit_ns) {
        if (err) atomicCAS(err, 0, PT_ERR_TIMEOUT_PEER);
        return;
      }
    }
    __nanosleep(64);
  }
}

// dst[0:bytes) = src[0:bytes), 16-byte vectors; loads bypass L1 so a peer's fresh data is seen.
// Eight independent loads are in flight per thread before the first store: a load over NVLink takes
// microseconds, and a copy that is limited to a few dozen CTAs (to leave the SMs to compute kernels)
// still has to cover the link's bandwidth-delay product.
__global__ void __launch_bounds__(256) copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long nvec) {
  constexpr int U = 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < nvec; i += U * stride) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                   : "l"(src + i + u * stride));
#pragma unroll
    for (int u = 0; u < U; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < nvec; i += stride) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i));
    dst[i] = v;
  }
}

}  // namespace symm
}  // namespace pt

// ctl_ptrs: host array of n device pointers (control blocks, own and peers').
PT_API int pt_symm_signal(const void* const* ctl_ptrs, int n, int index, unsigned value, void* stream) {
  using namespace pt::symm;
  if (n <= 0 || n > MAXW) return -1;
  PtrList l;
  for (int i = 0; i < n; ++i) l.p[i] = reinterpret_cast<unsigned*>(const_cast<void*>(ctl_ptrs[i]));
  signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(l, n, index, value);
  return (int)cudaGetLastError();
}

PT_API int pt_symm_wait(const void* ctl, int index, int count, unsigned value, void* stream) {
  using namespace pt::symm;
  if (count <= 0 || count > MAXW) return -1;
  wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const unsigned*>(ctl), index, count, value,
                                                                   pt::device_status_word());
  return (int)cudaGetLastError();
}

PT_API int pt_symm_copy(void* dst, const void* src, long long bytes, int max_ctas, void* stream) {
  using namespace pt::symm;
  if (bytes <= 0) return 0;
  if (bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -2;
  long long nvec = bytes / 16;
  long long blocks = (nvec + 255) / 256;
  int cap = max_ctas > 0 ? max_ctas : pt::sm_count() * 4;
  int grid = (int)(blocks < cap ? blocks : cap);
  copy_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<uint4*>(dst),
                                                                        reinterpret_cast<const uint4*>(src), nvec);
  return (int)cudaGetLastError();
}

// Sets this translation unit's copy of the peer-wait limit on the current device (see peer_wait.cuh).
extern "C" int pt_symm_set_wait_limit(unsigned long long ns) { return pt::set_peer_wait_limit_here(ns); }
