// RMSNorm (with fused residual add) and fused per-head QK-RMSNorm + rotary embedding, forward and
// backward. Memory-bound kernels: one 16-byte vector per thread per access, each tensor read once.
// They replace the Inductor-generated stage-1 region of the reference
// (pithtrain/models/qwen3_moe.py:156-168,188-202).
#include "elementwise.cuh"
#include "host_common.h"

namespace pt {

constexpr int NORM_THREADS = 256;

// y = (x [+ res]) * rstd * w ; optionally writes h = x + res and rstd.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int n_rows,
                   int H, float eps, int w_plus_one) {
  __shared__ float red[32];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (size_t)row * H;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        load8(xr + c * 8, v[i]);
        if (res) {
          float r[8];
          load8(res + (size_t)row * H + c * 8, r);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] += r[e];
          if (h_out) {
            // round to bf16 first so the norm sees exactly the stored residual stream
            store8(h_out + (size_t)row * H + c * 8, v[i]);
            load8(h_out + (size_t)row * H + c * 8, v[i]);
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
      }
    }
    ss = block_sum(ss, red);
    float rstd = rsqrtf(ss / H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        float wv[8], o[8];
        load8(w + c * 8, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd * (w_plus_one ? (1.f + wv[e]) : wv[e]);
        store8(y + (size_t)row * H + c * 8, o);
      }
    }
  }
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) [+ dh_extra]; dw partial per CTA (fp32).
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ dh_extra,
                   const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w,
                   const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int n_rows, int H, int w_plus_one) {
  __shared__ float red[32];
  const int nvec = H / 8;
  float dw[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dw[i][e] = 0.f;
  for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {
    float rstd = rstd_in[row];
    float xh[VPT][8], g[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        float wv[8];
        load8(h + (size_t)row * H + c * 8, xh[i]);
        load8(dy + (size_t)row * H + c * 8, g[i]);
        load8(w + c * 8, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[i][e] *= rstd;
          dw[i][e] += g[i][e] * xh[i][e];
          g[i][e] *= (w_plus_one ? (1.f + wv[e]) : wv[e]);
          dot += g[i][e] * xh[i][e];
        }
      }
    }
    dot = block_sum(dot, red) / H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd * (g[i][e] - xh[i][e] * dot);
        if (dh_extra) {
          float ex[8];
          load8(dh_extra + (size_t)row * H + c * 8, ex);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += ex[e];
        }
        store8(dx + (size_t)row * H + c * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float* p = dw_partial + (size_t)blockIdx.x * H + c * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) p[e] = dw[i][e];
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Fused per-head RMSNorm (optional) + rotate-half RoPE for q and k, reading the fused qkv GEMM output.
// A head of D elements is handled by D/16 lanes: lane `sub` owns elements [8 sub, 8 sub + 8) of the first
// half and their rotation partners in the second half, so every access is a 16-byte vector and the pair
// (i, i + D/2) never leaves the lane. A warp covers 32 / (D/16) heads. D in {64, 128}: PAIRS = D / 64.
// ----------------------------------------------------------------------------------------------
template <int LPH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPH / 2; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int PAIRS>
__global__ void __launch_bounds__(256)
qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                        __nv_bfloat16* __restrict__ k_out, const __nv_bfloat16* __restrict__ qw,
                        const __nv_bfloat16* __restrict__ kw, const __nv_bfloat16* __restrict__ cosb,
                        const __nv_bfloat16* __restrict__ sinb, const int* __restrict__ pos,
                        float* __restrict__ rstd_q, float* __restrict__ rstd_k, int n_tokens, int S,
                        int Hq, int Hkv, long long qkv_stride, float eps, int w_plus_one, int rot_dim) {
  constexpr int D = PAIRS * 64, HALF = D / 2, LPH = D / 16, HPW = 32 / LPH;
  const int lane = threadIdx.x & 31, sub = lane % LPH, i0 = sub * 8;
  const int heads = Hq + Hkv;
  const long long total = (long long)n_tokens * heads;
  const long long item = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * HPW + lane / LPH;
  const bool live = item < total;
  const long long it = live ? item : total - 1;
  const int tok = (int)(it / heads), hd = (int)(it % heads);
  const bool is_q = hd < Hq;
  const __nv_bfloat16* src = qkv + (size_t)tok * qkv_stride + (size_t)hd * D;  // k heads follow q heads
  __nv_bfloat16* dst = is_q ? q_out + ((size_t)tok * Hq + hd) * D : k_out + ((size_t)tok * Hkv + (hd - Hq)) * D;
  const __nv_bfloat16* wn = is_q ? qw : kw;
  const int p = pos ? pos[tok] : (tok % S);
  float a[8], b[8];
  load8(src + i0, a);
  load8(src + HALF + i0, b);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
  float rstd = 1.f;
  if (wn) {
    ss = group_sum<LPH>(ss);
    rstd = rsqrtf(ss / D + eps);
    if (live && sub == 0) {
      if (is_q) rstd_q[(size_t)tok * Hq + hd] = rstd;
      else rstd_k[(size_t)tok * Hkv + (hd - Hq)] = rstd;
    }
  }
  float wa[8], wb[8], c[8], sn[8];
  if (wn) {
    load8(wn + i0, wa);
    load8(wn + HALF + i0, wb);
  }
  const bool rotate = rot_dim == D;
  if (rotate) {
    load8(cosb + (size_t)p * D + i0, c);
    load8(sinb + (size_t)p * D + i0, sn);
  }
  float oa[8], ob[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float na = a[e] * rstd, nb = b[e] * rstd;
    if (wn) {
      float x = wa[e], y = wb[e];
      if (w_plus_one) { x += 1.f; y += 1.f; }
      na *= x; nb *= y;
    }
    // round like the unfused path (norm output is bf16 before the rotation)
    na = __bfloat162float(__float2bfloat16(na));
    nb = __bfloat162float(__float2bfloat16(nb));
    oa[e] = rotate ? na * c[e] - nb * sn[e] : na;
    ob[e] = rotate ? nb * c[e] + na * sn[e] : nb;
  }
  if (live) {
    store8(dst + i0, oa);
    store8(dst + HALF + i0, ob);
  }
}

template <int PAIRS>
__global__ void __launch_bounds__(256)
qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                        const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ dqkv,
                        const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                        const __nv_bfloat16* __restrict__ cosb, const __nv_bfloat16* __restrict__ sinb,
                        const int* __restrict__ pos, const float* __restrict__ rstd_q,
                        const float* __restrict__ rstd_k, float* __restrict__ dw_partial,
                        int n_tokens, int S, int Hq, int Hkv, long long qkv_stride, int w_plus_one) {
  constexpr int D = PAIRS * 64, HALF = D / 2, LPH = D / 16, HPW = 32 / LPH;
  __shared__ float acc[2 * D];  // weight-gradient sums of this CTA: q scales then k scales
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const int sub = lane % LPH, i0 = sub * 8;
  const int heads = Hq + Hkv;
  const long long total = (long long)n_tokens * heads;
  for (int cidx = threadIdx.x; cidx < 2 * D; cidx += blockDim.x) acc[cidx] = 0.f;
  __syncthreads();
  float dwq_a[8], dwq_b[8], dwk_a[8], dwk_b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) dwq_a[e] = dwq_b[e] = dwk_a[e] = dwk_b[e] = 0.f;
  for (long long base = ((long long)blockIdx.x * wpb + wib) * HPW; base < total; base += (long long)gridDim.x * wpb * HPW) {
    const long long item = base + lane / LPH;
    const bool live = item < total;
    const long long it = live ? item : total - 1;
    const int tok = (int)(it / heads), hd = (int)(it % heads);
    const bool is_q = hd < Hq;
    const __nv_bfloat16* g = is_q ? dq + ((size_t)tok * Hq + hd) * D : dk + ((size_t)tok * Hkv + (hd - Hq)) * D;
    const __nv_bfloat16* src = qkv + (size_t)tok * qkv_stride + (size_t)hd * D;
    __nv_bfloat16* dst = dqkv + (size_t)tok * qkv_stride + (size_t)hd * D;
    const __nv_bfloat16* wn = is_q ? qw : kw;
    const int p = pos ? pos[tok] : (tok % S);
    float ga[8], gb[8], c[8], sn[8], dna[8], dnb[8], xa[8], xb[8];
    load8(g + i0, ga);
    load8(g + HALF + i0, gb);
    load8(cosb + (size_t)p * D + i0, c);
    load8(sinb + (size_t)p * D + i0, sn);
    float rstd = 1.f;
    if (wn) rstd = is_q ? rstd_q[(size_t)tok * Hq + hd] : rstd_k[(size_t)tok * Hkv + (hd - Hq)];
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dna[e] = ga[e] * c[e] + gb[e] * sn[e];
      dnb[e] = gb[e] * c[e] - ga[e] * sn[e];
    }
    if (wn) {
      float wa[8], wb[8];
      load8(src + i0, xa);
      load8(src + HALF + i0, xb);
      load8(wn + i0, wa);
      load8(wn + HALF + i0, wb);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xa[e] *= rstd; xb[e] *= rstd;
        float x = wa[e], y = wb[e];
        if (w_plus_one) { x += 1.f; y += 1.f; }
        if (live) {
          if (is_q) { dwq_a[e] += dna[e] * xa[e]; dwq_b[e] += dnb[e] * xb[e]; }
          else { dwk_a[e] += dna[e] * xa[e]; dwk_b[e] += dnb[e] * xb[e]; }
        }
        dna[e] *= x; dnb[e] *= y;
        dot += dna[e] * xa[e] + dnb[e] * xb[e];
      }
      dot = group_sum<LPH>(dot) / D;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dna[e] = rstd * (dna[e] - xa[e] * dot);
        dnb[e] = rstd * (dnb[e] - xb[e] * dot);
      }
    }
    if (live) {
      store8(dst + i0, dna);
      store8(dst + HALF + i0, dnb);
    }
  }
  if (qw && dw_partial) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      atomicAdd(&acc[i0 + e], dwq_a[e]);
      atomicAdd(&acc[HALF + i0 + e], dwq_b[e]);
      atomicAdd(&acc[D + i0 + e], dwk_a[e]);
      atomicAdd(&acc[D + HALF + i0 + e], dwk_b[e]);
    }
    __syncthreads();
    for (int cidx = threadIdx.x; cidx < 2 * D; cidx += blockDim.x) dw_partial[(size_t)blockIdx.x * 2 * D + cidx] = acc[cidx];
  }
}

}  // namespace pt

using namespace pt;

PT_API int pt_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out,
                          float* rstd, int n_rows, int H, float eps, int w_plus_one, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_rows <= 0) return 0;
  if (H % 8 != 0 || H > 8 * NORM_THREADS * 4) return -1;
  int vpt = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
  int grid = n_rows < sm_count() * 8 ? n_rows : sm_count() * 8;
#define LAUNCH(V)                                                                                     \
  rmsnorm_fwd_kernel<V><<<grid, NORM_THREADS, 0, st>>>(                                               \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, \
      (__nv_bfloat16*)h_out, rstd, n_rows, H, eps, w_plus_one)
  switch (vpt) { case 1: LAUNCH(1); break; case 2: LAUNCH(2); break; case 3: LAUNCH(3); break; default: LAUNCH(4); }
#undef LAUNCH
  return (int)cudaGetLastError();
}

// dw_partial must hold [grid, H] floats where grid = pt_rmsnorm_bwd_grid(n_rows).
PT_API int pt_rmsnorm_bwd_grid(int n_rows) {
  int g = sm_count() * 4;
  return n_rows < g ? (n_rows > 0 ? n_rows : 1) : g;
}
PT_API int pt_rmsnorm_bwd(const void* dy, const void* dh_extra, const void* h, const void* w,
                          const float* rstd, void* dx, float* dw_partial, int n_rows, int H,
                          int w_plus_one, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_rows <= 0) return 0;
  if (H % 8 != 0 || H > 8 * NORM_THREADS * 4) return -1;
  int vpt = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
  int grid = pt_rmsnorm_bwd_grid(n_rows);
#define LAUNCH(V)                                                                                 \
  rmsnorm_bwd_kernel<V><<<grid, NORM_THREADS, 0, st>>>(                                           \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)dh_extra, (const __nv_bfloat16*)h,          \
      (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, dw_partial, n_rows, H, w_plus_one)
  switch (vpt) { case 1: LAUNCH(1); break; case 2: LAUNCH(2); break; case 3: LAUNCH(3); break; default: LAUNCH(4); }
#undef LAUNCH
  return (int)cudaGetLastError();
}

PT_API int pt_qk_norm_rope_fwd(const void* qkv, void* q_out, void* k_out, const void* qw,
                               const void* kw, const void* cosb, const void* sinb, const int* pos,
                               float* rstd_q, float* rstd_k, int n_tokens, int S, int Hq, int Hkv,
                               int D, long long qkv_stride, float eps, int w_plus_one, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_tokens <= 0) return 0;
  if (D != 64 && D != 128) return -1;
  const int heads_per_warp = 32 / (D / 16);
  long long warps = ((long long)n_tokens * (Hq + Hkv) + heads_per_warp - 1) / heads_per_warp;
  int grid = (int)((warps + 7) / 8);
  if (D == 128)
    qk_norm_rope_fwd_kernel<2><<<grid, 256, 0, st>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out,
        (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, (const __nv_bfloat16*)cosb, (const __nv_bfloat16*)sinb, pos,
        rstd_q, rstd_k, n_tokens, S, Hq, Hkv, qkv_stride, eps, w_plus_one, D);
  else
    qk_norm_rope_fwd_kernel<1><<<grid, 256, 0, st>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out,
        (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, (const __nv_bfloat16*)cosb, (const __nv_bfloat16*)sinb, pos,
        rstd_q, rstd_k, n_tokens, S, Hq, Hkv, qkv_stride, eps, w_plus_one, D);
  return (int)cudaGetLastError();
}

PT_API int pt_qk_norm_rope_bwd_grid() { return sm_count() * 4; }
// dw_partial: [grid, 2*D] floats (q weight grads then k weight grads per row); may be null when qw is null.
PT_API int pt_qk_norm_rope_bwd(const void* dq, const void* dk, const void* qkv, void* dqkv,
                               const void* qw, const void* kw, const void* cosb, const void* sinb,
                               const int* pos, const float* rstd_q, const float* rstd_k,
                               float* dw_partial, int n_tokens, int S, int Hq, int Hkv, int D,
                               long long qkv_stride, int w_plus_one, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_tokens <= 0) return 0;
  if (D != 64 && D != 128) return -1;
  int grid = pt_qk_norm_rope_bwd_grid();
  if (D == 128)
    qk_norm_rope_bwd_kernel<2><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)qkv,
        (__nv_bfloat16*)dqkv, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, (const __nv_bfloat16*)cosb,
        (const __nv_bfloat16*)sinb, pos, rstd_q, rstd_k, dw_partial, n_tokens, S, Hq, Hkv, qkv_stride, w_plus_one);
  else
    qk_norm_rope_bwd_kernel<1><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)qkv,
        (__nv_bfloat16*)dqkv, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, (const __nv_bfloat16*)cosb,
        (const __nv_bfloat16*)sinb, pos, rstd_q, rstd_k, dw_partial, n_tokens, S, Hq, Hkv, qkv_stride, w_plus_one);
  return (int)cudaGetLastError();
}

// ----------------------------------------------------------------------------------------------
// dst[c] += sum_g part[g, c]: finishes the per-block partial sums of a weight gradient (RMSNorm scale,
// QK-norm scales) and accumulates into the gradient buffer in one launch.
// ----------------------------------------------------------------------------------------------
namespace pt {
template <typename T>
__global__ void __launch_bounds__(128)
colsum_accumulate_kernel(const float* __restrict__ part, int G, int ld, int H, T* __restrict__ dst) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
  int g = 0;
  for (; g + 3 < G; g += 4) {
    acc0 += part[(size_t)g * ld + c];
    acc1 += part[(size_t)(g + 1) * ld + c];
    acc2 += part[(size_t)(g + 2) * ld + c];
    acc3 += part[(size_t)(g + 3) * ld + c];
  }
  for (; g < G; ++g) acc0 += part[(size_t)g * ld + c];
  const float s = (acc0 + acc1) + (acc2 + acc3);
  dst[c] = (T)((float)dst[c] + s);
}
}  // namespace pt

// part: G rows of pitch ld floats; columns [0, H) of it are summed into dst[0:H).
PT_API int pt_colsum_accumulate(const float* part, int G, int ld, int H, void* dst, int dst_fp32, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (G <= 0 || H <= 0) return 0;
  int grid = (H + 127) / 128;
  if (dst_fp32) pt::colsum_accumulate_kernel<float><<<grid, 128, 0, st>>>(part, G, ld, H, (float*)dst);
  else pt::colsum_accumulate_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(part, G, ld, H, (__nv_bfloat16*)dst);
  return (int)cudaGetLastError();
}
