// Optimizer-side kernels over flat parameter / gradient buffers: sum of squares for the global
// gradient norm (no fp32 copy of a 50 GB buffer), and fused AdamW on a flat region with the
// gradient scale (1/num_tokens x clip coefficient) read from device memory.
// They replace the per-parameter foreach kernels of the reference's optimizer step
// (pithtrain/tasks/pretrain_lm.py:125-153,393-405).
#include "elementwise.cuh"
#include "host_common.h"

namespace pt {

template <typename T>
__device__ __forceinline__ void load_as_float8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load_as_float8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) { load8(p, f); }
template <>
__device__ __forceinline__ void load_as_float8<float>(const float* p, float (&f)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void store_from_float8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store_from_float8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) { store8(p, f); }
template <>
__device__ __forceinline__ void store_from_float8<float>(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

template <typename T>
__global__ void __launch_bounds__(512)
sumsq_kernel(const T* __restrict__ x, long long nvec, double* __restrict__ partial) {
  __shared__ float red[32];
  float acc = 0.f;
  double total = 0.0;
  int it = 0;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    float f[8];
    load_as_float8<T>(x + v * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += f[e] * f[e];
    if (++it == 64) { total += acc; acc = 0.f; it = 0; }  // bound fp32 accumulation error
  }
  total += acc;
  float s = block_sum((float)total, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = (double)s;
}

// AdamW on a flat region. grad_scale (device float) multiplies the gradient first.
template <typename TP, typename TG>
__global__ void __launch_bounds__(256)
adamw_kernel(TP* __restrict__ p, const TG* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             long long nvec, const float* __restrict__ grad_scale, float lr, float b1, float b2, float eps,
             float wd, float bc1, float bc2) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float pf[8], gf[8], mf[8], vf[8];
    load_as_float8<TP>(p + i * 8, pf);
    load_as_float8<TG>(g + i * 8, gf);
    load_as_float8<float>(m + i * 8, mf);
    load_as_float8<float>(v + i * 8, vf);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float gg = gf[e] * gs;
      mf[e] = b1 * mf[e] + (1.f - b1) * gg;
      vf[e] = b2 * vf[e] + (1.f - b2) * gg * gg;
      float denom = sqrtf(vf[e] / bc2) + eps;
      pf[e] = pf[e] * (1.f - lr * wd) - lr * (mf[e] / bc1) / denom;
    }
    store_from_float8<TP>(p + i * 8, pf);
    store_from_float8<float>(m + i * 8, mf);
    store_from_float8<float>(v + i * 8, vf);
  }
}

// Muon momentum + Nesterov blend: buf = beta*buf + (1-beta)*g ; upd = (1-beta)*g + beta*buf (bf16 out).
template <typename TG, typename TB>
__global__ void __launch_bounds__(256)
muon_momentum_kernel(const TG* __restrict__ g, TB* __restrict__ buf, __nv_bfloat16* __restrict__ upd,
                     long long nvec, float beta, const float* __restrict__ grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.f;  // deferred 1/num_tokens and clip coefficient
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float gf[8], bf[8], uf[8];
    load_as_float8<TG>(g + i * 8, gf);
    load_as_float8<TB>(buf + i * 8, bf);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      gf[e] *= gs;
      bf[e] = beta * bf[e] + (1.f - beta) * gf[e];
      uf[e] = (1.f - beta) * gf[e] + beta * bf[e];
    }
    store_from_float8<TB>(buf + i * 8, bf);
    store8(upd + i * 8, uf);
  }
}

// w = w * decay + alpha * x  (bf16 weights, bf16 update)
__global__ void __launch_bounds__(256)
axpby_bf16_kernel(__nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ x, long long nvec,
                  float decay, float alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float wf[8], xf[8];
    load8(w + i * 8, wf);
    load8(x + i * 8, xf);
#pragma unroll
    for (int e = 0; e < 8; ++e) wf[e] = wf[e] * decay + alpha * xf[e];
    store8(w + i * 8, wf);
  }
}

}  // namespace pt

using namespace pt;

static inline int flat_grid(long long nvec) {
  long long want = (nvec + 255) / 256, cap = (long long)sm_count() * 16;
  return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

PT_API int pt_muon_momentum(const void* g, int g_fp32, void* buf, int buf_fp32, void* upd, long long numel,
                            float beta, const float* grad_scale, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (numel <= 0) return 0;
  if (numel % 8 != 0) return -1;
  long long nvec = numel / 8;
  int grid = flat_grid(nvec);
#define LAUNCH(TG, TB) muon_momentum_kernel<TG, TB><<<grid, 256, 0, st>>>((const TG*)g, (TB*)buf, (__nv_bfloat16*)upd, nvec, beta, grad_scale)
  if (g_fp32 && buf_fp32) LAUNCH(float, float);
  else if (g_fp32) LAUNCH(float, __nv_bfloat16);
  else if (buf_fp32) LAUNCH(__nv_bfloat16, float);
  else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return (int)cudaGetLastError();
}

PT_API int pt_axpby_bf16(void* w, const void* x, long long numel, float decay, float alpha, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (numel <= 0) return 0;
  if (numel % 8 != 0) return -1;
  long long nvec = numel / 8;
  axpby_bf16_kernel<<<flat_grid(nvec), 256, 0, st>>>((__nv_bfloat16*)w, (const __nv_bfloat16*)x, nvec, decay, alpha);
  return (int)cudaGetLastError();
}

PT_API int pt_sumsq_grid() { return sm_count() * 4; }
// partial: [pt_sumsq_grid()] doubles. numel must be a multiple of 8.
PT_API int pt_sumsq(const void* x, int is_fp32, long long numel, double* partial, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (numel % 8 != 0) return -1;
  int grid = pt_sumsq_grid();
  if (is_fp32) sumsq_kernel<float><<<grid, 512, 0, st>>>((const float*)x, numel / 8, partial);
  else sumsq_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>((const __nv_bfloat16*)x, numel / 8, partial);
  return (int)cudaGetLastError();
}

PT_API int pt_adamw(void* p, int p_fp32, const void* g, int g_fp32, float* m, float* v, long long numel,
                    const float* grad_scale, float lr, float b1, float b2, float eps, float wd, float bc1,
                    float bc2, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (numel <= 0) return 0;
  if (numel % 8 != 0) return -1;
  long long nvec = numel / 8;
  long long want = (nvec + 255) / 256, cap = (long long)sm_count() * 16;
  int grid = (int)(want < cap ? want : cap);
#define LAUNCH(TP, TG) adamw_kernel<TP, TG><<<grid, 256, 0, st>>>((TP*)p, (const TG*)g, m, v, nvec, grad_scale, lr, b1, b2, eps, wd, bc1, bc2)
  if (p_fp32 && g_fp32) LAUNCH(float, float);
  else if (p_fp32) LAUNCH(float, __nv_bfloat16);
  else if (g_fp32) LAUNCH(__nv_bfloat16, float);
  else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  return (int)cudaGetLastError();
}
