// Merge of two partial attention results over disjoint key sets (ring attention, one call per visited block):
//   lse' = log(exp(lse) + exp(lse_p)),  out' = out * exp(lse - lse') + o_p * exp(lse_p - lse')
// out [rows, H, D] fp32 is updated in place, the merged lse [B, H, S] fp32 is written to a second array; the partial
// o_p is bf16 or fp32 with a row pitch, lse_p [B, H, S] fp32. Rows whose two log-sum-exps are both -inf (no key seen
// yet) get out = 0, lse = -inf.
// One pass over the operands instead of the eight elementwise tensor ops of the restatement in
// ops/ring_attention.py: merge_partial (the reference does this step in pithtrain/operators/ring_attention.py:30-60).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "host_common.h"

namespace pt {

// One thread per 4 consecutive output elements of a (token, head) row; D % 4 == 0.
template <typename TP>
__global__ void merge_partial_kernel(float* __restrict__ out, const float* __restrict__ lse, const TP* __restrict__ o_p,
                                     const float* __restrict__ lse_p, long long rows, int S, int H, int D,
                                     long long ldp) {
  const int per_row = D / 4;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long rh = gid / per_row;  // (token, head)
  const int part = static_cast<int>(gid % per_row);
  if (rh >= rows * H) return;
  const long long row = rh / H;
  const int h = static_cast<int>(rh % H);
  const long long b = row / S, s = row % S;
  const long long li = (b * H + h) * S + s;
  const float a = lse[li], c = lse_p[li];
  const float m = fmaxf(a, c);
  float w_old = 0.f, w_new = 0.f;
  if (m != -INFINITY) {
    const float ea = __expf(a - m), ec = __expf(c - m);
    const float inv = 1.f / (ea + ec);
    w_old = ea * inv;
    w_new = ec * inv;
  }
  float4* op = reinterpret_cast<float4*>(out + (row * H + h) * D) + part;
  float4 o = *op;
  float p0, p1, p2, p3;
  if constexpr (sizeof(TP) == 2) {
    const uint2 raw = *reinterpret_cast<const uint2*>(o_p + row * ldp + (long long)h * D + part * 4);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    p0 = __low2float(lo); p1 = __high2float(lo); p2 = __low2float(hi); p3 = __high2float(hi);
  } else {
    const float4 raw = *reinterpret_cast<const float4*>(o_p + row * ldp + (long long)h * D + part * 4);
    p0 = raw.x; p1 = raw.y; p2 = raw.z; p3 = raw.w;
  }
  o.x = o.x * w_old + p0 * w_new;
  o.y = o.y * w_old + p1 * w_new;
  o.z = o.z * w_old + p2 * w_new;
  o.w = o.w * w_old + p3 * w_new;
  *op = o;
}

// The merged log-sum-exp goes to its own array: the D / 4 threads of a row above all read the old value.
__global__ void merge_lse_kernel(const float* __restrict__ lse, const float* __restrict__ lse_p, float* __restrict__ lse_out,
                                 long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float a = lse[i], c = lse_p[i];
  const float m = fmaxf(a, c);
  lse_out[i] = (m == -INFINITY) ? -INFINITY : m + __logf(__expf(a - m) + __expf(c - m));
}

}  // namespace pt

// out [B*S, H, D] fp32 (contiguous) and lse [B, H, S] fp32 are the running result; o_p [B*S, H*D] with row pitch ldp
// (elements; bf16 when p_fp32 == 0), lse_p [B, H, S] fp32. The output rows are merged in place from the old lse; the new
// log-sum-exp goes to lse_out [B, H, S] (a different array: the row threads read the old one).
PT_API int pt_merge_partial(void* out, const void* lse, const void* o_p, int p_fp32, const void* lse_p, void* lse_out, int B,
                            int S, int H, int D, long long ldp, void* stream_) {
  using namespace pt;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (B <= 0 || S <= 0 || H <= 0 || D <= 0) return 0;
  if (D % 4 != 0 || ldp % 4 != 0 || lse == lse_out) return -2;
  const long long rows = (long long)B * S;
  const long long threads = rows * H * (D / 4);
  const int block = 256;
  const long long grid = (threads + block - 1) / block;
  if (grid > 0x7fffffffLL) return -2;
  if (p_fp32)
    merge_partial_kernel<float><<<(unsigned)grid, block, 0, st>>>((float*)out, (const float*)lse, (const float*)o_p,
                                                                 (const float*)lse_p, rows, S, H, D, ldp);
  else
    merge_partial_kernel<__nv_bfloat16><<<(unsigned)grid, block, 0, st>>>((float*)out, (const float*)lse,
                                                                         (const __nv_bfloat16*)o_p, (const float*)lse_p, rows,
                                                                         S, H, D, ldp);
  const long long n = (long long)B * H * S;
  merge_lse_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const float*)lse, (const float*)lse_p, (float*)lse_out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
