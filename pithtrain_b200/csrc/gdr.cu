// Gated delta rule (Gated DeltaNet linear attention): the recurrence over chunks, forward and backward.
//
// The chunked form of the rule (the blocking of the library kernels the reference wraps,
// pithtrain/operators/gated_delta_rule.py:21-56) splits into algebra inside a chunk of C = 64 positions (batched
// matrix products and a triangular solve, done by the caller) and a sequential pass over the chunks that carries the
// [dk, dv] state S of every head:
//
//     v_new_n   = u_n - w_n S_n                 [C, dv]     value updates after what the state already explains
//     o_inter_n = qg_n S_n                      [C, dv]     contribution of the carried state to the outputs
//     S_{n+1}   = a_n S_n + kd_n^T v_new_n      [dk, dv]    decay by a_n = exp(sum of the chunk's log gates), then update
//
// with w, qg, kd [B,H,N,C,dk], u [B,H,N,C,dv], a [B,H,N] prepared by the caller in fp32. These kernels run that pass:
// one CTA per (batch, head, 32-column slice of the value dimension) -- the columns of S evolve independently, which is
// where the parallelism of a single sequence comes from -- with the state slice resident in shared memory for the whole
// walk. The forward stores every chunk's entry state (the backward needs it); the backward walks the chunks in reverse
// with dS resident and produces d_u directly and d_w, d_qg, d_kd, d_a as sums over the value slices (atomic adds into
// zeroed fp32 buffers: four-way contention at dv = 128).
//
// Plain fp32 FMA math (the products are [64 x 128] x [128 x 32]: a few MFLOP per chunk); the work list is launch- and
// latency-bound in its PyTorch form (one Python iteration and a dozen small launches per chunk), not FLOP-bound.
#include "host_common.h"

#include <cuda_runtime.h>

namespace pt {

constexpr int GD_C = 64;    // chunk length
constexpr int GD_VS = 32;   // value columns per CTA
constexpr int GD_THREADS = 256;

// out[r][v] (+)= sign * sum_k A[r][k] * S[k][v]   for r < 64, v < 32; A [64][DK] and S [DK][32] in shared memory.
// Thread layout: r = tid / 4, v-group = tid % 4 (8 columns each).
template <int DK>
__device__ __forceinline__ void rows_times_state(const float* __restrict__ A, const float* __restrict__ S, float (&acc)[8]) {
  const int r = threadIdx.x >> 2, vg = threadIdx.x & 3;
  const float* a = A + r * DK;
  const float* s = S + vg * 8;
#pragma unroll 4
  for (int k = 0; k < DK; ++k) {
    const float av = a[k];
    const float4 s0 = *reinterpret_cast<const float4*>(s + k * GD_VS);
    const float4 s1 = *reinterpret_cast<const float4*>(s + k * GD_VS + 4);
    acc[0] = fmaf(av, s0.x, acc[0]); acc[1] = fmaf(av, s0.y, acc[1]);
    acc[2] = fmaf(av, s0.z, acc[2]); acc[3] = fmaf(av, s0.w, acc[3]);
    acc[4] = fmaf(av, s1.x, acc[4]); acc[5] = fmaf(av, s1.y, acc[5]);
    acc[6] = fmaf(av, s1.z, acc[6]); acc[7] = fmaf(av, s1.w, acc[7]);
  }
}

// acc[j] = sum_c A[c][k] * V[c][v0 + j]   for one k (row of the state) and 16 columns; A [64][DK], V [64][32].
// Thread layout of the caller: k = tid / 2 (+128 per pass), half = tid % 2.
template <int DK>
__device__ __forceinline__ void cols_times_rows(const float* __restrict__ A, const float* __restrict__ V, int k, int v0,
                                                float sign, float (&acc)[16]) {
#pragma unroll 4
  for (int c = 0; c < GD_C; ++c) {
    const float av = sign * A[c * DK + k];
    const float* vrow = V + c * GD_VS + v0;
#pragma unroll
    for (int j = 0; j < 16; j += 4) {
      const float4 x = *reinterpret_cast<const float4*>(vrow + j);
      acc[j] = fmaf(av, x.x, acc[j]); acc[j + 1] = fmaf(av, x.y, acc[j + 1]);
      acc[j + 2] = fmaf(av, x.z, acc[j + 2]); acc[j + 3] = fmaf(av, x.w, acc[j + 3]);
    }
  }
}

// out[c][k] = sum_v X[c][v] * S[k][v] (32 columns of this slice), added atomically to global g[c][k].
template <int DK>
__device__ __forceinline__ void rows_times_state_t_atomic(const float* __restrict__ X, const float* __restrict__ S,
                                                          float sign, float* __restrict__ g) {
  // 64 x DK outputs over 256 threads: thread handles row c = tid / 4 and k = (tid % 4) + 4 * i
  const int c = threadIdx.x >> 2;
  const float* x = X + c * GD_VS;
  float xr[GD_VS];
#pragma unroll
  for (int v = 0; v < GD_VS; ++v) xr[v] = x[v];
  for (int k = (threadIdx.x & 3); k < DK; k += 4) {
    const float* s = S + k * GD_VS;
    float acc = 0.f;
#pragma unroll
    for (int v = 0; v < GD_VS; ++v) acc = fmaf(xr[v], s[v], acc);
    atomicAdd(g + c * DK + k, sign * acc);
  }
}

template <int DK>
__device__ __forceinline__ void load_tile(float* __restrict__ dst, const float* __restrict__ src, int n_floats) {
  for (int i = threadIdx.x * 4; i < n_floats; i += GD_THREADS * 4)
    *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
}

struct GdrArgs {
  const float *w, *u, *qg, *kd, *a;   // inputs (see the header comment)
  float *v_new, *o_inter, *states;    // forward outputs; `states` [B,H,N,dk,dv] = S_n at the entry of chunk n
  int BH, N, dv;
};

template <int DK>
__global__ void __launch_bounds__(GD_THREADS)
gdr_state_fwd_kernel(const GdrArgs p) {
  extern __shared__ float sm[];
  float* S = sm;                       // [DK][32]
  float* A = S + DK * GD_VS;           // [64][DK] staging for w / qg / kd
  float* V = A + GD_C * DK;            // [64][32] v_new
  const int bh = blockIdx.x, vs = blockIdx.y * GD_VS;
  const int r = threadIdx.x >> 2, vg = threadIdx.x & 3;
  for (int i = threadIdx.x; i < DK * GD_VS; i += GD_THREADS) S[i] = 0.f;
  __syncthreads();
  for (int n = 0; n < p.N; ++n) {
    const size_t ck = ((size_t)bh * p.N + n) * GD_C * DK;        // [C, dk] tiles
    const size_t cv = ((size_t)bh * p.N + n) * GD_C * p.dv;      // [C, dv] tiles
    // entry state of the chunk, for the backward
    {
      float* st = p.states + ((size_t)bh * p.N + n) * DK * p.dv;
      for (int i = threadIdx.x; i < DK * GD_VS / 4; i += GD_THREADS) {
        const int k = i / (GD_VS / 4), q4 = i % (GD_VS / 4);
        *reinterpret_cast<float4*>(st + (size_t)k * p.dv + vs + 4 * q4) = *reinterpret_cast<const float4*>(S + k * GD_VS + 4 * q4);
      }
    }
    // v_new = u - w S
    load_tile<DK>(A, p.w + ck, GD_C * DK);
    __syncthreads();
    float acc[8];
    {
      const float* urow = p.u + cv + (size_t)r * p.dv + vs + vg * 8;
      const float4 u0 = *reinterpret_cast<const float4*>(urow), u1 = *reinterpret_cast<const float4*>(urow + 4);
      float neg[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      rows_times_state<DK>(A, S, neg);
      acc[0] = u0.x - neg[0]; acc[1] = u0.y - neg[1]; acc[2] = u0.z - neg[2]; acc[3] = u0.w - neg[3];
      acc[4] = u1.x - neg[4]; acc[5] = u1.y - neg[5]; acc[6] = u1.z - neg[6]; acc[7] = u1.w - neg[7];
    }
    {
      float* vrow = V + r * GD_VS + vg * 8;
      *reinterpret_cast<float4*>(vrow) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(vrow + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      float* g = p.v_new + cv + (size_t)r * p.dv + vs + vg * 8;
      *reinterpret_cast<float4*>(g) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(g + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    __syncthreads();
    // o_inter = qg S
    load_tile<DK>(A, p.qg + ck, GD_C * DK);
    __syncthreads();
    {
      float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      rows_times_state<DK>(A, S, o);
      float* g = p.o_inter + cv + (size_t)r * p.dv + vs + vg * 8;
      *reinterpret_cast<float4*>(g) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4*>(g + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
    __syncthreads();
    // S = a S + kd^T v_new
    load_tile<DK>(A, p.kd + ck, GD_C * DK);
    __syncthreads();
    const float an = p.a[(size_t)bh * p.N + n];
    for (int k = threadIdx.x >> 1; k < DK; k += GD_THREADS / 2) {
      const int v0 = (threadIdx.x & 1) * 16;
      float s[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) s[j] = an * S[k * GD_VS + v0 + j];
      cols_times_rows<DK>(A, V, k, v0, 1.f, s);
#pragma unroll
      for (int j = 0; j < 16; ++j) S[k * GD_VS + v0 + j] = s[j];  // each (k, v) belongs to one thread
    }
    __syncthreads();
  }
}

struct GdrBwdArgs {
  const float *w, *qg, *kd, *a, *v_new, *states;   // saved by the forward
  const float *d_o, *d_vnew_ext;                   // incoming gradients [B,H,N,C,dv]
  float *d_u, *d_w, *d_qg, *d_kd, *d_a;            // d_u written; the others zeroed by the caller, summed over slices
  int BH, N, dv;
};

template <int DK>
__global__ void __launch_bounds__(GD_THREADS)
gdr_state_bwd_kernel(const GdrBwdArgs p) {
  extern __shared__ float sm[];
  float* dS = sm;                      // [DK][32] gradient w.r.t. the state after the current chunk
  float* Sn = dS + DK * GD_VS;         // [DK][32] entry state of the chunk
  float* A = Sn + DK * GD_VS;          // [64][DK]
  float* X = A + GD_C * DK;            // [64][32] d_vnew
  float* Y = X + GD_C * GD_VS;         // [64][32] d_o / v_new
  __shared__ float red[GD_THREADS / 32];
  const int bh = blockIdx.x, vs = blockIdx.y * GD_VS;
  const int r = threadIdx.x >> 2, vg = threadIdx.x & 3;
  for (int i = threadIdx.x; i < DK * GD_VS; i += GD_THREADS) dS[i] = 0.f;
  __syncthreads();
  for (int n = p.N - 1; n >= 0; --n) {
    const size_t ck = ((size_t)bh * p.N + n) * GD_C * DK;
    const size_t cv = ((size_t)bh * p.N + n) * GD_C * p.dv;
    const float an = p.a[(size_t)bh * p.N + n];
    // entry state slice
    {
      const float* st = p.states + ((size_t)bh * p.N + n) * DK * p.dv;
      for (int i = threadIdx.x; i < DK * GD_VS / 4; i += GD_THREADS) {
        const int k = i / (GD_VS / 4), q4 = i % (GD_VS / 4);
        *reinterpret_cast<float4*>(Sn + k * GD_VS + 4 * q4) = *reinterpret_cast<const float4*>(st + (size_t)k * p.dv + vs + 4 * q4);
      }
    }
    // d_vnew = d_vnew_ext + kd dS
    load_tile<DK>(A, p.kd + ck, GD_C * DK);
    __syncthreads();
    {
      const float* e = p.d_vnew_ext + cv + (size_t)r * p.dv + vs + vg * 8;
      const float4 e0 = *reinterpret_cast<const float4*>(e), e1 = *reinterpret_cast<const float4*>(e + 4);
      float acc[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
      rows_times_state<DK>(A, dS, acc);
      float* xr = X + r * GD_VS + vg * 8;
      *reinterpret_cast<float4*>(xr) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(xr + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      float* g = p.d_u + cv + (size_t)r * p.dv + vs + vg * 8;  // d_u = d_vnew
      *reinterpret_cast<float4*>(g) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(g + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      // v_new slice for d_kd
      const float* vn = p.v_new + cv + (size_t)r * p.dv + vs + vg * 8;
      float* yr = Y + r * GD_VS + vg * 8;
      *reinterpret_cast<float4*>(yr) = *reinterpret_cast<const float4*>(vn);
      *reinterpret_cast<float4*>(yr + 4) = *reinterpret_cast<const float4*>(vn + 4);
    }
    __syncthreads();
    // d_kd[c][k] += sum_v v_new[c][v] dS[k][v];  d_w[c][k] -= sum_v d_vnew[c][v] S_n[k][v]
    rows_times_state_t_atomic<DK>(Y, dS, 1.f, p.d_kd + ck);
    rows_times_state_t_atomic<DK>(X, Sn, -1.f, p.d_w + ck);
    // d_a += <dS, S_n>
    {
      float part = 0.f;
      for (int i = threadIdx.x; i < DK * GD_VS; i += GD_THREADS) part = fmaf(dS[i], Sn[i], part);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int i = 0; i < GD_THREADS / 32; ++i) tot += red[i];
      atomicAdd(p.d_a + (size_t)bh * p.N + n, tot);
    }
    // d_o slice into Y (v_new no longer needed)
    __syncthreads();
    {
      const float* e = p.d_o + cv + (size_t)r * p.dv + vs + vg * 8;
      float* yr = Y + r * GD_VS + vg * 8;
      *reinterpret_cast<float4*>(yr) = *reinterpret_cast<const float4*>(e);
      *reinterpret_cast<float4*>(yr + 4) = *reinterpret_cast<const float4*>(e + 4);
    }
    __syncthreads();
    // d_qg[c][k] += sum_v d_o[c][v] S_n[k][v]
    rows_times_state_t_atomic<DK>(Y, Sn, 1.f, p.d_qg + ck);
    // dS = a dS + qg^T d_o - w^T d_vnew
    load_tile<DK>(A, p.qg + ck, GD_C * DK);  // kd tile in A is no longer read by anyone past the barrier above
    __syncthreads();
    float keep[(DK + GD_THREADS / 2 - 1) / (GD_THREADS / 2)][16];
    {
      int it = 0;
      for (int k = threadIdx.x >> 1; k < DK; k += GD_THREADS / 2, ++it) {
        const int v0 = (threadIdx.x & 1) * 16;
#pragma unroll
        for (int j = 0; j < 16; ++j) keep[it][j] = an * dS[k * GD_VS + v0 + j];
        cols_times_rows<DK>(A, Y, k, v0, 1.f, keep[it]);
      }
    }
    __syncthreads();
    load_tile<DK>(A, p.w + ck, GD_C * DK);
    __syncthreads();
    {
      int it = 0;
      for (int k = threadIdx.x >> 1; k < DK; k += GD_THREADS / 2, ++it) {
        const int v0 = (threadIdx.x & 1) * 16;
        cols_times_rows<DK>(A, X, k, v0, -1.f, keep[it]);
#pragma unroll
        for (int j = 0; j < 16; ++j) dS[k * GD_VS + v0 + j] = keep[it][j];
      }
    }
    __syncthreads();
  }
}

}  // namespace pt

using namespace pt;

// Forward pass over the chunks. All tensors fp32 and contiguous: w, qg, kd [BH, N, 64, dk]; u, v_new, o_inter
// [BH, N, 64, dv]; a [BH, N]; states [BH, N, dk, dv]. dk in {64, 128}, dv a multiple of 32.
PT_API int pt_gdr_state_fwd(const float* w, const float* u, const float* qg, const float* kd, const float* a, float* v_new,
                            float* o_inter, float* states, int BH, int N, int dk, int dv, void* stream_) {
  if (BH <= 0 || N <= 0 || dv % GD_VS != 0 || (dk != 64 && dk != 128)) return -2;
  GdrArgs p{w, u, qg, kd, a, v_new, o_inter, states, BH, N, dv};
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  dim3 grid(BH, dv / GD_VS);
  const int smem = (dk * GD_VS + GD_C * dk + GD_C * GD_VS) * (int)sizeof(float);
  if (dk == 128) {
    static bool cfg = false;
    if (!cfg) { if (cudaFuncSetAttribute(gdr_state_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4; cfg = true; }
    gdr_state_fwd_kernel<128><<<grid, GD_THREADS, smem, st>>>(p);
  } else {
    static bool cfg = false;
    if (!cfg) { if (cudaFuncSetAttribute(gdr_state_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4; cfg = true; }
    gdr_state_fwd_kernel<64><<<grid, GD_THREADS, smem, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Backward pass (reverse walk). d_w, d_qg, d_kd [BH, N, 64, dk] and d_a [BH, N] must be zeroed by the caller (they
// are sums over the value slices); d_u [BH, N, 64, dv] is written.
PT_API int pt_gdr_state_bwd(const float* w, const float* qg, const float* kd, const float* a, const float* v_new,
                            const float* states, const float* d_o, const float* d_vnew_ext, float* d_u, float* d_w,
                            float* d_qg, float* d_kd, float* d_a, int BH, int N, int dk, int dv, void* stream_) {
  if (BH <= 0 || N <= 0 || dv % GD_VS != 0 || (dk != 64 && dk != 128)) return -2;
  GdrBwdArgs p{w, qg, kd, a, v_new, states, d_o, d_vnew_ext, d_u, d_w, d_qg, d_kd, d_a, BH, N, dv};
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  dim3 grid(BH, dv / GD_VS);
  const int smem = (2 * dk * GD_VS + GD_C * dk + 2 * GD_C * GD_VS) * (int)sizeof(float);
  if (dk == 128) {
    static bool cfg = false;
    if (!cfg) { if (cudaFuncSetAttribute(gdr_state_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4; cfg = true; }
    gdr_state_bwd_kernel<128><<<grid, GD_THREADS, smem, st>>>(p);
  } else {
    static bool cfg = false;
    if (!cfg) { if (cudaFuncSetAttribute(gdr_state_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4; cfg = true; }
    gdr_state_bwd_kernel<64><<<grid, GD_THREADS, smem, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
