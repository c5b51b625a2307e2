// MoE routing and data-movement kernels, all sized from device-side counts (no host sync):
//   router_topk  : softmax -> top-k (-> renormalise) or top-k -> softmax, fwd + bwd
//   route_count / route_place : stable counting sort of (token, slot) pairs by local expert into a
//                  16-row-aligned grouped layout: offs[E+1], row_of_slot, slot_of_row
//   gather_rows  : build the expert-sorted activation matrix (pad rows zeroed)
//   combine      : out[t] = residual[t] + sum_j w[t,j] * y[row_of_slot[t,j]]   (gather-reduce, no atomics)
//   swiglu fwd / fused backward (also emits routing-weight grads and the weight-scaled activation
//                  that the down-projection wgrad consumes)
// These replace the reference's Triton scatter kernels and compiled stage-5 region
// (pithtrain/operators/token_scatter.py:38-153, pithtrain/models/qwen3_moe.py:81-89,229-245,
// pithtrain/operators/silu_mul.py:28-87, pithtrain/operators/clamped_swiglu.py:18-89).
#include "elementwise.cuh"
#include <mutex>

#include "host_common.h"
#include "no_alloc.h"
#include "ptx.cuh"

namespace pt {

// ----------------------------------------------------------------------------------------------
// Router: one warp per token, E <= 512 experts (E/32 values per lane), k <= 16.
// mode 0: p = softmax(logits); pick top-k of p; w = p[idx] (/ sum if renorm) * scale
// mode 1: pick top-k of logits; w = softmax over the k picked logits * scale   (GPT-OSS)
// ----------------------------------------------------------------------------------------------
constexpr int MAX_EPL = 16;  // experts per lane

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(256)
router_topk_fwd_kernel(const T* __restrict__ logits, float* __restrict__ probs,
                       int* __restrict__ topk_idx, float* __restrict__ topk_w, int n, int E, int k,
                       int mode, int renorm, float scale) {
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= n) return;
  const int epl = (E + 31) / 32;
  float v[MAX_EPL];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAX_EPL; ++j) {
    int e = lane + 32 * j;
    v[j] = (j < epl && e < E) ? ld_as_float(logits + (size_t)tok * E + e) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  if (mode == 0) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_EPL; ++j) {
      v[j] = (v[j] == -INFINITY) ? 0.f : __expf(v[j] - mx);
      s += v[j];
    }
    s = warp_sum(s);
    float inv = 1.f / s;
#pragma unroll
    for (int j = 0; j < MAX_EPL; ++j) {
      int e = lane + 32 * j;
      v[j] *= inv;
      if (j < epl && e < E && probs) probs[(size_t)tok * E + e] = v[j];
      if (!(j < epl && e < E)) v[j] = -1.f;  // never selected
    }
  }
  // iterative arg-max; ties resolve to the lowest expert index
  float picked_w[16];
  int picked_i[16];
  float wsum = 0.f;
  for (int t = 0; t < k; ++t) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAX_EPL; ++j) {
      int e = lane + 32 * j;
      if (j < epl && e < E && (v[j] > best)) { best = v[j]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    picked_w[t] = best;
    picked_i[t] = bi;
    wsum += best;
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < MAX_EPL; ++j) if (j == (bi >> 5)) v[j] = -INFINITY;
    }
  }
  if (mode == 1) {
    // softmax over the k selected logits (picked_w[0] is the maximum)
    float s = 0.f;
    const float top = picked_w[0];
    for (int t = 0; t < k; ++t) { picked_w[t] = __expf(picked_w[t] - top); s += picked_w[t]; }
    for (int t = 0; t < k; ++t) picked_w[t] = picked_w[t] / s * scale;
  } else {
    float mul = renorm ? scale / wsum : scale;
    for (int t = 0; t < k; ++t) picked_w[t] *= mul;
  }
  if (lane == 0) {
    for (int t = 0; t < k; ++t) {
      topk_idx[(size_t)tok * k + t] = picked_i[t];
      topk_w[(size_t)tok * k + t] = picked_w[t];
    }
  }
}

// d_logits from d_topk_w (and an optional dense d_probs, e.g. from a load-balance loss).
template <typename T>
__global__ void __launch_bounds__(256)
router_topk_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ topk_idx,
                       const float* __restrict__ topk_w, const float* __restrict__ d_topk_w,
                       const float* __restrict__ d_probs, T* __restrict__ d_logits, int n, int E,
                       int k, int mode, int renorm, float scale) {
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= n) return;
  const int epl = (E + 31) / 32;
  float dp[MAX_EPL];
#pragma unroll
  for (int j = 0; j < MAX_EPL; ++j) {
    int e = lane + 32 * j;
    dp[j] = (mode == 0 && d_probs && j < epl && e < E) ? d_probs[(size_t)tok * E + e] : 0.f;
  }
  if (mode == 0) {
    // w_j = scale * p_j / s (renorm) or scale * p_j
    float s = 0.f, dot = 0.f;
    for (int t = 0; t < k; ++t) {
      float w = topk_w[(size_t)tok * k + t], dw = d_topk_w[(size_t)tok * k + t];
      int e = topk_idx[(size_t)tok * k + t];
      s += probs[(size_t)tok * E + e];
      dot += dw * w;
    }
    for (int t = 0; t < k; ++t) {
      int e = topk_idx[(size_t)tok * k + t];
      float dw = d_topk_w[(size_t)tok * k + t];
      float g = renorm ? (dw * scale - dot) / s : dw * scale;
      if ((e & 31) == lane) {
#pragma unroll
        for (int j = 0; j < MAX_EPL; ++j) if (j == (e >> 5)) dp[j] += g;
      }
    }
    float pd = 0.f;
    float p[MAX_EPL];
#pragma unroll
    for (int j = 0; j < MAX_EPL; ++j) {
      int e = lane + 32 * j;
      p[j] = (j < epl && e < E) ? probs[(size_t)tok * E + e] : 0.f;
      pd += p[j] * dp[j];
    }
    pd = warp_sum(pd);
#pragma unroll
    for (int j = 0; j < MAX_EPL; ++j) {
      int e = lane + 32 * j;
      if (j < epl && e < E) d_logits[(size_t)tok * E + e] = (T)(p[j] * (dp[j] - pd));
    }
  } else {
    float dot = 0.f;
    for (int t = 0; t < k; ++t) dot += d_topk_w[(size_t)tok * k + t] * topk_w[(size_t)tok * k + t];
#pragma unroll
    for (int j = 0; j < MAX_EPL; ++j) dp[j] = 0.f;
    for (int t = 0; t < k; ++t) {
      int e = topk_idx[(size_t)tok * k + t];
      float w = topk_w[(size_t)tok * k + t], dw = d_topk_w[(size_t)tok * k + t];
      // w = scale * softmax  ->  dlogit = w * (dw - sum(dw * w) / scale)
      float g = w * (dw - dot / scale);
      if ((e & 31) == lane) {
#pragma unroll
        for (int j = 0; j < MAX_EPL; ++j) if (j == (e >> 5)) dp[j] += g;
      }
    }
#pragma unroll
    for (int j = 0; j < MAX_EPL; ++j) {
      int e = lane + 32 * j;
      if (j < epl && e < E) d_logits[(size_t)tok * E + e] = (T)dp[j];
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Stable counting sort by expert. One CTA per expert scans all slots in order, so ranks inside a
// group follow slot order: deterministic, no atomics. eids < 0 or >= E are skipped.
// ----------------------------------------------------------------------------------------------
constexpr int ROUTE_THREADS = 512;

__global__ void __launch_bounds__(ROUTE_THREADS)
route_count_kernel(const int* __restrict__ eids, const int* __restrict__ n_ptr, int n_max, int E,
                   int* __restrict__ counts) {
  __shared__ float red[32];
  const int e = blockIdx.x;
  const int n = n_ptr ? min(*n_ptr, n_max) : n_max;
  int c = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) c += (eids[i] == e);
  float tot = block_sum((float)c, red);
  if (threadIdx.x == 0) counts[e] = (int)(tot + 0.5f);
}

__global__ void __launch_bounds__(ROUTE_THREADS)
route_place_kernel(const int* __restrict__ eids, const int* __restrict__ n_ptr, int n_max, int E,
                   int align, const int* __restrict__ counts, int* __restrict__ offs,
                   int* __restrict__ row_of_slot, int* __restrict__ slot_of_row, int r_cap,
                   int* __restrict__ err) {
  __shared__ int warp_tot[ROUTE_THREADS / 32];
  __shared__ int base_sh;
  const int e = blockIdx.x;
  const int n = n_ptr ? min(*n_ptr, n_max) : n_max;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (threadIdx.x == 0) {
    int b = 0;
    for (int j = 0; j < e; ++j) b += (counts[j] + align - 1) / align * align;
    base_sh = b;
    offs[e] = b;
    if (e == E - 1) {
      int end = b + (counts[e] + align - 1) / align * align;
      offs[E] = end;
      if (end > r_cap && err) atomicCAS(err, 0, PT_ERR_CAPACITY);
    }
  }
  __syncthreads();
  int base = base_sh;
  const int my_rows = (counts[e] + align - 1) / align * align;
  if (base + my_rows > r_cap) return;  // overflow reported by the last block
  int running = 0;
  for (int start = 0; start < n; start += blockDim.x) {
    int i = start + threadIdx.x;
    bool hit = (i < n) && (eids[i] == e);
    unsigned m = __ballot_sync(0xffffffffu, hit);
    int before = __popc(m & ((1u << lane) - 1));
    if (lane == 0) warp_tot[w] = __popc(m);
    __syncthreads();
    int woff = 0, tot = 0;
    for (int j = 0; j < nw; ++j) { int t = warp_tot[j]; if (j < w) woff += t; tot += t; }
    if (hit) {
      int r = base + running + woff + before;
      row_of_slot[i] = r;
      slot_of_row[r] = i;
    }
    running += tot;
    __syncthreads();
  }
  // pad rows of this group
  for (int r = base + counts[e] + threadIdx.x; r < base + my_rows; r += blockDim.x) slot_of_row[r] = -1;
}

// Slots that were skipped (eid < 0) get row -1; rows past offs[E] get slot -1.
__global__ void route_fill_kernel(const int* __restrict__ eids, const int* __restrict__ n_ptr,
                                  int n_max, int E, const int* __restrict__ offs,
                                  int* __restrict__ row_of_slot, int* __restrict__ slot_of_row,
                                  int r_cap) {
  const int n = n_ptr ? min(*n_ptr, n_max) : n_max;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_max) {
    if (i >= n || eids[i] < 0 || eids[i] >= E) row_of_slot[i] = -1;
  }
  int end = min(offs[E], r_cap);
  if (i < r_cap && i >= end) slot_of_row[i] = -1;
}

// ----------------------------------------------------------------------------------------------
// gather_rows: dst[r] = src[idx[r] / div]  (zero row when idx[r] < 0). One warp per row, 16B vectors.
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx, int div,
                   __nv_bfloat16* __restrict__ dst, const int* __restrict__ n_rows_ptr,
                   int n_rows_max, int H, long long src_stride) {
  const int n_rows = n_rows_ptr ? min(*n_rows_ptr, n_rows_max) : n_rows_max;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < n_rows; r += gridDim.x * wpb) {
    int s = idx[r];
    uint4* d = reinterpret_cast<uint4*>(dst + (size_t)r * H);
    if (s < 0) {
      for (int c = lane; c < H / 8; c += 32) d[c] = make_uint4(0, 0, 0, 0);
    } else {
      const uint4* p = reinterpret_cast<const uint4*>(src + (size_t)(s / div) * src_stride);
      for (int c = lane; c < H / 8; c += 32) d[c] = p[c];
    }
  }
}

// ----------------------------------------------------------------------------------------------
// combine: out[t] = (res ? res[t] : 0) + sum_{j<k, row>=0} (w ? w[t,j] : 1) * y[row_of_slot[t*k+j]]
// One warp per token; fp32 accumulation; k rows gathered per token.
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_of_slot,
               const float* __restrict__ w, const __nv_bfloat16* __restrict__ res,
               __nv_bfloat16* __restrict__ out, const int* __restrict__ n_ptr, int n_max, int k,
               int H) {
  const int n = n_ptr ? min(*n_ptr, n_max) : n_max;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < n; t += gridDim.x * wpb) {
    for (int c0 = lane * 8; c0 < H; c0 += 256) {
      float acc[8];
      if (res) load8(res + (size_t)t * H + c0, acc);
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      }
      for (int j = 0; j < k; ++j) {
        int r = row_of_slot[(size_t)t * k + j];
        if (r < 0) continue;
        float wt = w ? w[(size_t)t * k + j] : 1.f;
        float v[8];
        load8(y + (size_t)r * H + c0, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += wt * v[e];
      }
      store8(out + (size_t)t * H + c0, acc);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// SwiGLU. gu is [R, 2I]: gate = cols [0,I), up = cols [I,2I) (interleaved = 0) or gate = even cols,
// up = odd cols (interleaved = 1, GPT-OSS). limit > 0 enables the clamped form
//   gc = min(g, limit), uc = clamp(u, +-limit), act = (uc + 1) * gc * sigmoid(alpha * gc).
// Plain form: act = silu(g) * u.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void swiglu_point(float g, float u, float alpha, float limit, float& act,
                                             float& dact_dg, float& dact_du) {
  if (limit > 0.f) {
    float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
    float sg = 1.f / (1.f + __expf(-alpha * gc));
    float glu = gc * sg;
    act = (uc + 1.f) * glu;
    float dglu = sg + alpha * gc * sg * (1.f - sg);
    dact_dg = (g <= limit) ? (uc + 1.f) * dglu : 0.f;
    dact_du = (u >= -limit && u <= limit) ? glu : 0.f;
  } else {
    float sg = 1.f / (1.f + __expf(-g));
    act = g * sg * u;
    dact_dg = u * (sg + g * sg * (1.f - sg));
    dact_du = g * sg;
  }
}

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                  const int* __restrict__ n_rows_ptr, int n_rows_max, int I, int interleaved,
                  float alpha, float limit) {
  const int n_rows = n_rows_ptr ? min(*n_rows_ptr, n_rows_max) : n_rows_max;
  const int vec_per_row = I / 8;
  const long long total = (long long)n_rows * vec_per_row;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total;
       v += (long long)gridDim.x * blockDim.x) {
    int r = (int)(v / vec_per_row), c = (int)(v % vec_per_row) * 8;
    float g[8], u[8], o[8];
    const __nv_bfloat16* row = gu + (size_t)r * 2 * I;
    if (!interleaved) {
      load8(row + c, g);
      load8(row + I + c, u);
    } else {
      float a[8], b[8];
      load8(row + 2 * c, a);
      load8(row + 2 * c + 8, b);
#pragma unroll
      for (int e = 0; e < 4; ++e) { g[e] = a[2 * e]; u[e] = a[2 * e + 1]; g[e + 4] = b[2 * e]; u[e + 4] = b[2 * e + 1]; }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) { float dg, du; swiglu_point(g[e], u[e], alpha, limit, o[e], dg, du); }
    store8(act + (size_t)r * I + c, o);
  }
}

// Backward with optional per-row routing weight. One warp per row.
//   dact_in      : gradient w.r.t. the (unweighted) activation            [R, I]
//   row_w        : per-row routing weight (nullable -> 1)                  [R]
//   dgu          : out, gradient w.r.t. gu = row_w * dact_in * d act/d gu  [R, 2I]
//   act_scaled   : out (nullable), row_w * act  — wgrad operand of the down projection
//   d_row_w      : out (nullable), <dact_in, act>
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact_in,
                  const float* __restrict__ row_w, __nv_bfloat16* __restrict__ dgu,
                  __nv_bfloat16* __restrict__ act_scaled, float* __restrict__ d_row_w,
                  const int* __restrict__ n_rows_ptr, int n_rows_max, int I, int interleaved,
                  float alpha, float limit, const int* __restrict__ slot_of_row) {
  const int n_rows = n_rows_ptr ? min(*n_rows_ptr, n_rows_max) : n_rows_max;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < n_rows; r += gridDim.x * wpb) {
    // with slot_of_row, row_w and d_row_w are indexed by the row's (token, slot) index instead of the row
    const int widx = slot_of_row ? slot_of_row[r] : r;
    const float wt = row_w ? (widx >= 0 ? row_w[widx] : 0.f) : 1.f;
    const __nv_bfloat16* row = gu + (size_t)r * 2 * I;
    __nv_bfloat16* drow = dgu + (size_t)r * 2 * I;
    float dot = 0.f;
    for (int c = lane * 8; c < I; c += 256) {
      float g[8], u[8], d[8], a[8], dg[8], du[8];
      if (!interleaved) {
        load8(row + c, g);
        load8(row + I + c, u);
      } else {
        float x[8], y[8];
        load8(row + 2 * c, x);
        load8(row + 2 * c + 8, y);
#pragma unroll
        for (int e = 0; e < 4; ++e) { g[e] = x[2 * e]; u[e] = x[2 * e + 1]; g[e + 4] = y[2 * e]; u[e + 4] = y[2 * e + 1]; }
      }
      load8(dact_in + (size_t)r * I + c, d);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float pg, pu;
        swiglu_point(g[e], u[e], alpha, limit, a[e], pg, pu);
        dot += d[e] * a[e];
        dg[e] = wt * d[e] * pg;
        du[e] = wt * d[e] * pu;
        a[e] *= wt;
      }
      if (!interleaved) {
        store8(drow + c, dg);
        store8(drow + I + c, du);
      } else {
        float x[8], y[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) { x[2 * e] = dg[e]; x[2 * e + 1] = du[e]; y[2 * e] = dg[e + 4]; y[2 * e + 1] = du[e + 4]; }
        store8(drow + 2 * c, x);
        store8(drow + 2 * c + 8, y);
      }
      if (act_scaled) store8(act_scaled + (size_t)r * I + c, a);
    }
    if (d_row_w) {
      dot = warp_sum(dot);
      if (lane == 0 && widx >= 0) d_row_w[widx] = dot;
    }
  }
}


// ----------------------------------------------------------------------------------------------
// Per-expert biases on expert-sorted rows (GPT-OSS). Takes the role of the reference's
// pithtrain/operators/indexed_bias_add.py (forward :54-83, segmented bias gradient :20-51).
//   indexed_bias_add: out[r] = x[r] + bias[group(r)], group(r) found by binary search in offs; one warp per row.
//   segment_sum:      out[g, c] = sum over rows of group g of x[r, c] * (row_w ? row_w[r] : 1), fp32, no atomics:
//                     one CTA per (group, 256-column slab), rows walked in order (deterministic).
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ int group_of_row(const int* __restrict__ offs, int E, int r) {
  int lo = 0, hi = E - 1;  // largest g with offs[g] <= r (rows past offs[E] map to the last group)
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (offs[mid] <= r) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(256)
indexed_bias_add_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias,
                        const int* __restrict__ offs, int E, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ n_rows_ptr, int n_rows_max, int H) {
  const int n_rows = n_rows_ptr ? min(*n_rows_ptr, n_rows_max) : n_rows_max;
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < n_rows; r += gridDim.x * wpb) {
    const int g = group_of_row(offs, E, r);
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)r * H);
    const uint4* br = reinterpret_cast<const uint4*>(bias + (size_t)g * H);
    uint4* orow = reinterpret_cast<uint4*>(out + (size_t)r * H);
    for (int c = lane; c < H / 8; c += 32) {
      const uint4 a = xr[c], b = br[c];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 u = unpack_bf16x2(aw[i]), v = unpack_bf16x2(bw[i]);
        o[i] = pack_bf16x2(u.x + v.x, u.y + v.y);
      }
      orow[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
segment_sum_kernel(const T* __restrict__ x, const float* __restrict__ row_w, const int* __restrict__ offs,
                   float* __restrict__ out, int H) {
  const int g = blockIdx.x;
  const int c = (blockIdx.y * 128 + threadIdx.x) * 2;
  if (c >= H) return;
  const int r0 = offs[g], r1 = offs[g + 1];
  float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
  int r = r0;
  for (; r + 1 < r1; r += 2) {
    float2 u, v;
    if constexpr (sizeof(T) == 2) {
      u = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + (size_t)r * H + c));
      v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + (size_t)(r + 1) * H + c));
    } else {
      u = *reinterpret_cast<const float2*>(x + (size_t)r * H + c);
      v = *reinterpret_cast<const float2*>(x + (size_t)(r + 1) * H + c);
    }
    const float wu = row_w ? row_w[r] : 1.f, wv = row_w ? row_w[r + 1] : 1.f;
    a0 = fmaf(u.x, wu, a0); a1 = fmaf(u.y, wu, a1);
    b0 = fmaf(v.x, wv, b0); b1 = fmaf(v.y, wv, b1);
  }
  if (r < r1) {
    float2 u;
    if constexpr (sizeof(T) == 2) u = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + (size_t)r * H + c));
    else u = *reinterpret_cast<const float2*>(x + (size_t)r * H + c);
    const float wu = row_w ? row_w[r] : 1.f;
    a0 = fmaf(u.x, wu, a0); a1 = fmaf(u.y, wu, a1);
  }
  *reinterpret_cast<float2*>(out + (size_t)g * H + c) = make_float2(a0 + b0, a1 + b1);
}

}  // namespace pt

using namespace pt;

static inline int grid_for(long long work_items, int per_block, int cap_mult = 8) {
  long long g = (work_items + per_block - 1) / per_block;
  long long cap = (long long)sm_count() * cap_mult;
  if (g > cap) g = cap;
  return g < 1 ? 1 : (int)g;
}

PT_API int pt_router_topk_fwd(const void* logits, int logits_fp32, float* probs, int* topk_idx,
                              float* topk_w, int n, int E, int k, int mode, int renorm, float scale,
                              void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n <= 0) return 0;
  if (E > 32 * MAX_EPL || k > 16 || k > E) return -1;
  int grid = (n + 7) / 8;
  if (logits_fp32)
    router_topk_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)logits, probs, topk_idx, topk_w, n, E, k, mode, renorm, scale);
  else
    router_topk_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)logits, probs, topk_idx, topk_w, n, E, k, mode, renorm, scale);
  return (int)cudaGetLastError();
}

PT_API int pt_router_topk_bwd(const float* probs, const int* topk_idx, const float* topk_w,
                              const float* d_topk_w, const float* d_probs, void* d_logits,
                              int dlogits_fp32, int n, int E, int k, int mode, int renorm,
                              float scale, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n <= 0) return 0;
  if (E > 32 * MAX_EPL || k > 16) return -1;
  int grid = (n + 7) / 8;
  if (dlogits_fp32)
    router_topk_bwd_kernel<float><<<grid, 256, 0, st>>>(probs, topk_idx, topk_w, d_topk_w, d_probs, (float*)d_logits, n, E, k, mode, renorm, scale);
  else
    router_topk_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(probs, topk_idx, topk_w, d_topk_w, d_probs, (__nv_bfloat16*)d_logits, n, E, k, mode, renorm, scale);
  return (int)cudaGetLastError();
}

// ----------------------------------------------------------------------------------------------
// Routing sort, chunked form: O(n) work instead of one scan of all slots per expert.
//   hist : every warp owns a chunk of ROUTE_CHUNK consecutive slots and counts experts in shared memory
//   scan : per expert, exclusive prefix over the chunks (slot order) and the aligned group offsets
//   place: every warp walks its chunk in slot order; match.any groups the lanes of one expert, so a
//          slot's row is offs[e] + (slots of e in earlier chunks) + (earlier slots of e in this chunk)
// The result is the same stable order as the per-expert kernels above.
// ----------------------------------------------------------------------------------------------
constexpr int ROUTE_CHUNK = 512;
constexpr int ROUTE_WARPS = 4;
constexpr int ROUTE_MAX_E_SMEM = 1024;

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_hist_kernel(const int* __restrict__ eids, const int* __restrict__ n_ptr, int n_max, int E,
                  int* __restrict__ hist /* [chunks, E] */) {
  extern __shared__ int sh[];  // [ROUTE_WARPS][E]
  const int n = n_ptr ? min(*n_ptr, n_max) : n_max;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * ROUTE_WARPS + w;
  int* my = sh + w * E;
  for (int e = lane; e < E; e += 32) my[e] = 0;
  __syncwarp();
  const int begin = chunk * ROUTE_CHUNK, end = min(begin + ROUTE_CHUNK, n);
  for (int i = begin + lane; i < end; i += 32) {
    int e = eids[i];
    if (e >= 0 && e < E) atomicAdd(&my[e], 1);
  }
  __syncwarp();
  const int chunks = (n_max + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  if (chunk < chunks)
    for (int e = lane; e < E; e += 32) hist[(long long)chunk * E + e] = my[e];
}

__global__ void __launch_bounds__(1024)
route_scan_kernel(int* __restrict__ hist, int chunks, int E, int align, int* __restrict__ offs, int r_cap,
                  int* __restrict__ err) {
  __shared__ int padded[ROUTE_MAX_E_SMEM];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      int v = hist[(long long)c * E + e];
      hist[(long long)c * E + e] = run;
      run += v;
    }
    padded[e] = (run + align - 1) / align * align;
    hist[(long long)chunks * E + e] = run;  // total per expert, kept after the chunk rows
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int b = 0;
    for (int e = 0; e < E; ++e) { offs[e] = b; b += padded[e]; }
    offs[E] = b;
    if (b > r_cap && err) atomicCAS(err, 0, PT_ERR_CAPACITY);
  }
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_place_chunk_kernel(const int* __restrict__ eids, const int* __restrict__ n_ptr, int n_max, int E,
                         const int* __restrict__ hist, const int* __restrict__ offs,
                         int* __restrict__ row_of_slot, int* __restrict__ slot_of_row, int r_cap) {
  extern __shared__ int sh[];  // [ROUTE_WARPS][E] running position per expert
  const int n = n_ptr ? min(*n_ptr, n_max) : n_max;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * ROUTE_WARPS + w;
  const int chunks = (n_max + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  if (offs[E] > r_cap) return;  // capacity overflow was reported by the scan
  int* run = sh + w * E;
  if (chunk < chunks)
    for (int e = lane; e < E; e += 32) run[e] = offs[e] + hist[(long long)chunk * E + e];
  __syncwarp();
  const int begin = chunk * ROUTE_CHUNK, end = min(begin + ROUTE_CHUNK, n);
  for (int start = begin; start < end; start += 32) {
    const int i = start + lane;
    int e = (i < end) ? eids[i] : -1;
    const bool valid = e >= 0 && e < E;
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? e : -1);
    int base = valid ? run[e] : 0;
    __syncwarp();
    if (valid) {
      const int r = base + __popc(peers & ((1u << lane) - 1));
      row_of_slot[i] = r;
      slot_of_row[r] = i;
      if ((peers & ((1u << lane) - 1)) == 0) run[e] = base + __popc(peers);  // first lane of the group
    } else if (i < end) {
      row_of_slot[i] = -1;
    }
    __syncwarp();
  }
  // slots past the device-side count
  const int hard_end = min(begin + ROUTE_CHUNK, n_max);
  for (int i = max(begin, n) + lane; i < hard_end; i += 32) row_of_slot[i] = -1;
}

// Pad rows of every group and the rows past the last group get slot -1.
__global__ void route_pad_kernel(const int* __restrict__ hist_totals, const int* __restrict__ offs, int E,
                                 int* __restrict__ slot_of_row, int r_cap) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= r_cap) return;
  const int end = min(offs[E], r_cap);
  if (r >= end) { slot_of_row[r] = -1; return; }
  // binary search for the group of row r
  int lo = 0, hi = E - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (offs[mid] <= r) lo = mid; else hi = mid - 1;
  }
  if (r >= offs[lo] + hist_totals[lo]) slot_of_row[r] = -1;
}

// Stable sort of n slots by expert id into groups aligned to `align` rows.
//   counts [E] scratch, offs [E+1], row_of_slot [n_max], slot_of_row [r_cap].
//   With counts_len >= (ceil(n_max / 512) + 1) * E the chunked O(n) kernels run (4 launches), else the
//   per-expert kernels (3 launches, counts_len >= E).
PT_API int pt_route_sort(const int* eids, const int* n_ptr, int n_max, int E, int align,
                         int* counts, long long counts_len, int* offs, int* row_of_slot, int* slot_of_row, int r_cap,
                         void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (E <= 0) return -1;
  const int chunks = (n_max + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  if (counts_len >= (long long)(chunks + 1) * E && E <= ROUTE_MAX_E_SMEM && n_max > 0) {
    // chunked sort; `counts` is the [chunks + 1, E] workspace
    const int blocks = (chunks + ROUTE_WARPS - 1) / ROUTE_WARPS;
    const size_t smem = (size_t)ROUTE_WARPS * E * sizeof(int);
    route_hist_kernel<<<blocks, ROUTE_WARPS * 32, smem, st>>>(eids, n_ptr, n_max, E, counts);
    route_scan_kernel<<<1, 1024, 0, st>>>(counts, chunks, E, align, offs, r_cap, device_status_word());
    route_place_chunk_kernel<<<blocks, ROUTE_WARPS * 32, smem, st>>>(eids, n_ptr, n_max, E, counts, offs, row_of_slot,
                                                                     slot_of_row, r_cap);
    if (r_cap > 0)
      route_pad_kernel<<<(r_cap + 255) / 256, 256, 0, st>>>(counts + (long long)chunks * E, offs, E, slot_of_row, r_cap);
    return (int)cudaGetLastError();
  }
  route_count_kernel<<<E, ROUTE_THREADS, 0, st>>>(eids, n_ptr, n_max, E, counts);
  route_place_kernel<<<E, ROUTE_THREADS, 0, st>>>(eids, n_ptr, n_max, E, align, counts, offs,
                                                  row_of_slot, slot_of_row, r_cap, device_status_word());
  int m = n_max > r_cap ? n_max : r_cap;
  route_fill_kernel<<<(m + 255) / 256, 256, 0, st>>>(eids, n_ptr, n_max, E, offs, row_of_slot, slot_of_row, r_cap);
  return (int)cudaGetLastError();
}

// ----------------------------------------------------------------------------------------------
// Routing sort for callers that must not allocate (declaration and contract: no_alloc.h).
// ----------------------------------------------------------------------------------------------
// Per-expert counters of the no-allocation variant. In host code this name is only a handle for
// the runtime, not a device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) int g_route_counts_scratch[PT_ROUTE_SORT_NOALLOC_MAX_EXPERTS];

namespace {
constexpr int kNoAllocMaxDevices = 64;
int* g_route_counts_addr[kNoAllocMaxDevices] = {nullptr};
std::mutex g_route_counts_mu;

// Device address of the scratch on the current device; resolved once per device.
int route_counts_scratch(int** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoAllocMaxDevices) return -1;
  std::lock_guard<std::mutex> lk(g_route_counts_mu);
  if (!g_route_counts_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_route_counts_scratch);
    if (e != cudaSuccess) {
      fprintf(stderr, "[pithtrain_b200] cudaGetSymbolAddress(route counters) failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return (int)e;
    }
    g_route_counts_addr[dev] = static_cast<int*>(p);
  }
  *out = g_route_counts_addr[dev];
  return 0;
}
}  // namespace

PT_API int pt_route_sort_noalloc(const int* eids, int n, int E, int align, int* offs, int* row_of_slot,
                                 int* slot_of_row, int r_cap, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (E <= 0 || n < 0 || align <= 0 || r_cap < 0 || !eids || !offs || !row_of_slot || !slot_of_row) return -1;
  if (E > PT_ROUTE_SORT_NOALLOC_MAX_EXPERTS) {
    fprintf(stderr, "[pithtrain_b200] pt_route_sort_noalloc: %d experts exceed the static scratch (max %d)\n", E,
            PT_ROUTE_SORT_NOALLOC_MAX_EXPERTS);
    return -2;
  }
  int* counts = nullptr;
  int rc = route_counts_scratch(&counts);
  if (rc != 0) return rc;
  // every counter in [0, E) is overwritten by the count kernel, nothing has to be cleared first
  route_count_kernel<<<E, ROUTE_THREADS, 0, st>>>(eids, nullptr, n, E, counts);
  route_place_kernel<<<E, ROUTE_THREADS, 0, st>>>(eids, nullptr, n, E, align, counts, offs, row_of_slot,
                                                  slot_of_row, r_cap, nullptr);
  int m = n > r_cap ? n : r_cap;
  if (m > 0)
    route_fill_kernel<<<(m + 255) / 256, 256, 0, st>>>(eids, nullptr, n, E, offs, row_of_slot, slot_of_row, r_cap);
  return (int)cudaGetLastError();
}

PT_API int pt_gather_rows(const void* src, const int* idx, int div, void* dst, const int* n_rows_ptr,
                          int n_rows_max, int H, long long src_stride, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_rows_max <= 0) return 0;
  if (H % 8 != 0) return -1;
  gather_rows_kernel<<<grid_for(n_rows_max, 8, 16), 256, 0, st>>>((const __nv_bfloat16*)src, idx, div,
      (__nv_bfloat16*)dst, n_rows_ptr, n_rows_max, H, src_stride);
  return (int)cudaGetLastError();
}

PT_API int pt_combine(const void* y, const int* row_of_slot, const float* w, const void* res, void* out,
                      const int* n_ptr, int n_max, int k, int H, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_max <= 0) return 0;
  if (H % 8 != 0) return -1;
  combine_kernel<<<grid_for(n_max, 8, 16), 256, 0, st>>>((const __nv_bfloat16*)y, row_of_slot, w,
      (const __nv_bfloat16*)res, (__nv_bfloat16*)out, n_ptr, n_max, k, H);
  return (int)cudaGetLastError();
}

PT_API int pt_swiglu_fwd(const void* gu, void* act, const int* n_rows_ptr, int n_rows_max, int I,
                         int interleaved, float alpha, float limit, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_rows_max <= 0) return 0;
  if (I % 8 != 0) return -1;
  swiglu_fwd_kernel<<<grid_for((long long)n_rows_max * (I / 8), 256, 16), 256, 0, st>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, n_rows_ptr, n_rows_max, I, interleaved, alpha, limit);
  return (int)cudaGetLastError();
}

PT_API int pt_swiglu_bwd(const void* gu, const void* dact, const float* row_w, void* dgu,
                         void* act_scaled, float* d_row_w, const int* n_rows_ptr, int n_rows_max,
                         int I, int interleaved, float alpha, float limit, const int* slot_of_row, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_rows_max <= 0) return 0;
  if (I % 8 != 0) return -1;
  swiglu_bwd_kernel<<<grid_for(n_rows_max, 8, 16), 256, 0, st>>>((const __nv_bfloat16*)gu,
      (const __nv_bfloat16*)dact, row_w, (__nv_bfloat16*)dgu, (__nv_bfloat16*)act_scaled, d_row_w,
      n_rows_ptr, n_rows_max, I, interleaved, alpha, limit, slot_of_row);
  return (int)cudaGetLastError();
}

// out[r] = x[r] + bias[group(r)] for the first n rows (device-side count optional); x, bias, out bf16, H % 8 == 0;
// out may alias x.
PT_API int pt_indexed_bias_add(const void* x, const void* bias, const int* offs, int E, void* out, const int* n_rows_ptr,
                               int n_rows_max, int H, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (n_rows_max <= 0) return 0;
  if (H % 8 != 0 || E <= 0) return -1;
  indexed_bias_add_kernel<<<grid_for(n_rows_max, 8, 16), 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)bias,
                                                                       offs, E, (__nv_bfloat16*)out, n_rows_ptr, n_rows_max, H);
  return (int)cudaGetLastError();
}

// out[g, :] = sum of rows [offs[g], offs[g+1]) of x (bf16 when x_fp32 == 0, else fp32), optionally weighted per row;
// out fp32 [E, H], H even.
PT_API int pt_segment_sum(const void* x, int x_fp32, const float* row_w, const int* offs, int E, float* out, int H,
                          void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  if (E <= 0 || H <= 0) return 0;
  if (H % 2 != 0) return -1;
  dim3 grid(E, (H / 2 + 127) / 128);
  if (x_fp32) segment_sum_kernel<float><<<grid, 128, 0, st>>>((const float*)x, row_w, offs, out, H);
  else segment_sum_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, row_w, offs, out, H);
  return (int)cudaGetLastError();
}
