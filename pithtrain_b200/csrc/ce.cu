// Fused cross-entropy over bf16 logits: per-row online softmax, per-token loss, and the logits are
// overwritten in place by d loss / d logits = softmax - onehot (zero for ignored rows), so the
// [tokens, vocab] matrix is materialised exactly once. Same contract as the reference's Triton
// kernel (pithtrain/operators/cross_entropy.py:15-125).
#include "elementwise.cuh"
#include "host_common.h"

namespace pt {

constexpr int CE_THREADS = 1024;

__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                     float* __restrict__ loss, int n, int V, long long ld, int ignore_index) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (row >= n) return;
  __nv_bfloat16* x = logits + (size_t)row * ld;
  const long long label = labels[row];
  const int nvec = V / 8;
  if (label == ignore_index) {
    for (int c = threadIdx.x; c < nvec; c += CE_THREADS) *reinterpret_cast<uint4*>(x + c * 8) = make_uint4(0, 0, 0, 0);
    for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) x[c] = __float2bfloat16(0.f);
    if (threadIdx.x == 0) loss[row] = 0.f;
    return;
  }
  // pass 1: online max / sum-exp
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
    float v[8];
    load8(x + c * 8, v);
    float lm = v[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) lm = fmaxf(lm, v[e]);
    float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += __expf(v[e] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    float v = __bfloat162float(x[c]);
    float nm = fmaxf(m, v);
    s = s * __expf(m - nm) + __expf(v - nm);
    m = nm;
  }
  float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  float gs = block_sum(s, red);
  float lse = gm + __logf(gs);
  float xl = __bfloat162float(x[label]);
  __syncthreads();  // everyone has read x[label] before it is overwritten
  if (threadIdx.x == 0) loss[row] = lse - xl;
  // pass 2: gradient in place
  for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
    float v[8];
    load8(x + c * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[e] = __expf(v[e] - lse);
      if (c * 8 + e == label) v[e] -= 1.f;
    }
    store8(x + c * 8, v);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    float v = __expf(__bfloat162float(x[c]) - lse);
    if (c == label) v -= 1.f;
    x[c] = __float2bfloat16(v);
  }
}

// x *= s[0] over a flat bf16 buffer (s on the device).
__global__ void scale_bf16_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ s, long long nvec) {
  const float sc = *s;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    float f[8];
    load8(x + v * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] *= sc;
    store8(x + v * 8, f);
  }
}

}  // namespace pt

using namespace pt;

PT_API int pt_cross_entropy(void* logits, const long long* labels, float* loss, int n, int V,
                            long long ld, int ignore_index, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n <= 0) return 0;
  if (ld % 8 != 0) return -1;
  cross_entropy_kernel<<<n, CE_THREADS, 0, st>>>((__nv_bfloat16*)logits, labels, loss, n, V, ld, ignore_index);
  return (int)cudaGetLastError();
}

PT_API int pt_scale_bf16(void* x, const float* s, long long numel, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (numel <= 0) return 0;
  if (numel % 8 != 0) return -1;
  long long nvec = numel / 8;
  long long g = (nvec + 255) / 256, cap = (long long)sm_count() * 16;
  scale_bf16_kernel<<<(int)(g < cap ? g : cap), 256, 0, st>>>((__nv_bfloat16*)x, s, nvec);
  return (int)cudaGetLastError();
}
