#include "host_common.h"

#include <mutex>

namespace pt {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
  });
  return fn;
}

constexpr int kMaxDevices = 16;
int* g_status[kMaxDevices] = {nullptr};
int g_sms[kMaxDevices] = {0};
std::mutex g_mu;

CUtensorMapDataType to_cu(TmDtype dt) {
  switch (dt) {
    case TM_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case TM_F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case TM_U8: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case TM_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case TM_I32: return CU_TENSOR_MAP_DATA_TYPE_INT32;
  }
  return CU_TENSOR_MAP_DATA_TYPE_UINT8;
}
int elem_size(TmDtype dt) {
  switch (dt) {
    case TM_BF16: case TM_F16: return 2;
    case TM_F32: case TM_I32: return 4;
    case TM_U8: return 1;
  }
  return 1;
}
CUtensorMapSwizzle to_cu(TmSwizzle s) {
  switch (s) {
    case TM_SW_NONE: return CU_TENSOR_MAP_SWIZZLE_NONE;
    case TM_SW_32: return CU_TENSOR_MAP_SWIZZLE_32B;
    case TM_SW_64: return CU_TENSOR_MAP_SWIZZLE_64B;
    case TM_SW_128: return CU_TENSOR_MAP_SWIZZLE_128B;
  }
  return CU_TENSOR_MAP_SWIZZLE_NONE;
}
}  // namespace

int* device_status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    if (cudaMalloc(&g_status[dev], 64) != cudaSuccess) return nullptr;
    cudaMemset(g_status[dev], 0, 64);
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sms[dev] = n > 0 ? n : 148;
  }
  return g_sms[dev];
}

int encode_tmap_2d(CUtensorMap* out, const void* base, TmDtype dt, uint64_t rows, uint64_t cols,
                   uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, TmSwizzle sw) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * (uint64_t)elem_size(dt)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, to_cu(dt), 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, to_cu(sw), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[pithtrain_b200] cuTensorMapEncodeTiled(2d) failed: %d base=%p rows=%llu cols=%llu "
            "ld=%llu box=%ux%u\n",
            (int)r, base, (unsigned long long)rows, (unsigned long long)cols,
            (unsigned long long)ld_elems, box_rows, box_cols);
    return (int)r;
  }
  return 0;
}

int encode_tmap_3d(CUtensorMap* out, const void* base, TmDtype dt, uint64_t d2, uint64_t rows,
                   uint64_t cols, uint64_t ld_elems, uint64_t ld2_elems, uint32_t box_d2,
                   uint32_t box_rows, uint32_t box_cols, TmSwizzle sw) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return -1;
  cuuint64_t dims[3] = {cols, rows, d2};
  cuuint64_t strides[2] = {ld_elems * (uint64_t)elem_size(dt), ld2_elems * (uint64_t)elem_size(dt)};
  cuuint32_t box[3] = {box_cols, box_rows, box_d2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, to_cu(dt), 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, to_cu(sw), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[pithtrain_b200] cuTensorMapEncodeTiled(3d) failed: %d\n", (int)r);
    return (int)r;
  }
  return 0;
}

}  // namespace pt

// Read-and-clear the status word of the current device (synchronises the device).
PT_API int pt_status_fetch_and_clear() {
  int* w = pt::device_status_word();
  if (!w) return -1;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) cudaMemset(w, 0, sizeof(int));
  return v;
}

PT_API int pt_sm_count() { return pt::sm_count(); }

extern "C" int pt_ep_set_wait_limit(unsigned long long ns);
extern "C" int pt_fsdp_set_wait_limit(unsigned long long ns);
extern "C" int pt_symm_set_wait_limit(unsigned long long ns);

// Limit (nanoseconds) of every wait on another GPU's flag, on the current device; the default is 2 s.
PT_API int pt_set_peer_wait_limit_ns(long long ns) {
  if (ns <= 0) return -2;
  const unsigned long long v = static_cast<unsigned long long>(ns);
  return (pt_ep_set_wait_limit(v) | pt_fsdp_set_wait_limit(v) | pt_symm_set_wait_limit(v)) == 0 ? 0 : -1;
}
