// FP8 (e4m3) quantizers with power-of-two (E8M0-representable) scales.
//
// Recipe, per group of values (a 1x128 row segment for activations and gradients, a 128x128 tile
// for weights):
//   a     = max(float(max|x|), 1e-4)
//   s_in  = a * (1/448)
//   scale = 2^ceil(log2 s_in), never below 2^-126        (exact powers of two stay unchanged)
//   q     = e4m3(float(x) * (1/scale))                   (1/scale is exact: an exponent flip)
// which is the recipe of pithtrain/operators/deepgemm_quantize.py:36-83 of the reference; the
// reference's five Triton kernels (:91-201, :341-426, :490-572, :637-706, :764-843) collapse into
// the two kernels below because the GEMM consumes row scales k-block-major and takes weights in
// both orientations from one launch.
//
// Layouts produced here are the ones gemm_fp8.cu consumes:
//   rows   : q [R, K] uint8 row-major; scales [ceil(K/128), ld_s] float, k-block-major, so the 128
//            epilogue threads of a tile read 128 consecutive floats per k-block.
//   blocks : q [G, N, K] and qT [G, K, N] uint8; scales [G, ceil(N/128), ceil(K/128)] and the
//            transposed [G, ceil(K/128), ceil(N/128)].
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "host_common.h"

namespace pt {

__device__ __forceinline__ void e8m0_scale(float amax, float& scale, float& rcp) {
  float a = fmaxf(amax, 1e-4f);
  float s_in = a * (1.0f / 448.0f);
  uint32_t bits = __float_as_uint(s_in);
  uint32_t e = bits >> 23;  // sign is 0
  if (bits & 0x7fffffu) e += 1;
  if (e < 1u) e = 1u;
  if (e > 254u) e = 254u;
  scale = __uint_as_float(e << 23);
  rcp = __uint_as_float((254u - e) << 23);
}

__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// One half-warp (16 lanes x 8 elements) per 1x128 segment. `idx` (optional) gathers source rows;
// a negative index yields a zero row (scale of the 1e-4 floor).
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ idx, int div,
                  const int* __restrict__ n_rows_dev, int R, int K, uint8_t* __restrict__ q,
                  float* __restrict__ s, long long ld_s) {
  const int kblocks = (K + 127) >> 7;
  const int rows = n_rows_dev ? min(*n_rows_dev, R) : R;
  const long long total = (long long)rows * kblocks;
  const int sub = threadIdx.x & 15;
  const uint32_t half_mask = 0xffffu << (threadIdx.x & 16);  // the two half-warps may leave the loop apart
  for (long long seg = (long long)blockIdx.x * 16 + (threadIdx.x >> 4); seg < total;
       seg += (long long)gridDim.x * 16) {
    const int row = (int)(seg / kblocks), kb = (int)(seg - (long long)row * kblocks);
    const int col = kb * 128 + sub * 8;
    int src = idx ? idx[row] : row;
    if (idx && src >= 0 && div > 1) src /= div;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (src >= 0 && col < K) {
      const __nv_bfloat16* p = x + (long long)src * ldx + col;
      if (col + 8 <= K) {
        uint4 u = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(h[i]);
          v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
      } else {
        for (int i = 0; i < 8 && col + i < K; ++i) v[i] = __bfloat162float(p[i]);
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(half_mask, amax, o, 16));
    float scale, rcp;
    e8m0_scale(amax, scale, rcp);
    if (col < K) {
      uint2 out;
      out.x = cvt_e4m3x4(v[0] * rcp, v[1] * rcp, v[2] * rcp, v[3] * rcp);
      out.y = cvt_e4m3x4(v[4] * rcp, v[5] * rcp, v[6] * rcp, v[7] * rcp);
      uint8_t* qp = q + (long long)row * K + col;
      if (col + 8 <= K) {
        *reinterpret_cast<uint2*>(qp) = out;
      } else {
        const uint8_t* b = reinterpret_cast<const uint8_t*>(&out);
        for (int i = 0; i < 8 && col + i < K; ++i) qp[i] = b[i];
      }
    }
    if (sub == 0) s[(long long)kb * ld_s + row] = scale;
  }
}

// One CTA (256 threads) per 128x128 tile of W[g]; writes the tile in both orientations.
__global__ void __launch_bounds__(256)
quant_block_kernel(const __nv_bfloat16* __restrict__ w, int N, int K, uint8_t* __restrict__ q,
                   uint8_t* __restrict__ qt, float* __restrict__ s, float* __restrict__ st) {
  __shared__ float red[8];
  __shared__ __align__(16) uint8_t tile[128][128 + 16];
  const int g = blockIdx.z, nb = blockIdx.y, kb = blockIdx.x;
  const int nblocks = gridDim.y, kblocks = gridDim.x;
  const __nv_bfloat16* wg = w + (long long)g * N * K;
  const int tr = threadIdx.x >> 4, tc = (threadIdx.x & 15) * 8;
  float v[8][8];
  float amax = 0.f;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const int n = nb * 128 + p * 16 + tr, k = kb * 128 + tc;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[p][i] = 0.f;
    if (n < N && k < K) {
      const __nv_bfloat16* src = wg + (long long)n * K + k;
      if (k + 8 <= K && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
        uint4 u = *reinterpret_cast<const uint4*>(src);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(h[i]);
          v[p][2 * i] = f.x; v[p][2 * i + 1] = f.y;
        }
      } else {
        for (int i = 0; i < 8 && k + i < K; ++i) v[p][i] = __bfloat162float(src[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[p][i]));
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  float scale, rcp;
  e8m0_scale(amax, scale, rcp);
  if (threadIdx.x == 0) {
    s[((long long)g * nblocks + nb) * kblocks + kb] = scale;
    if (st) st[((long long)g * kblocks + kb) * nblocks + nb] = scale;
  }
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    uint2 out;
    out.x = cvt_e4m3x4(v[p][0] * rcp, v[p][1] * rcp, v[p][2] * rcp, v[p][3] * rcp);
    out.y = cvt_e4m3x4(v[p][4] * rcp, v[p][5] * rcp, v[p][6] * rcp, v[p][7] * rcp);
    const int r = p * 16 + tr;
    *reinterpret_cast<uint2*>(&tile[r][tc]) = out;
    const int n = nb * 128 + r, k = kb * 128 + tc;
    if (n < N && k < K) {
      uint8_t* dst = q + ((long long)g * N + n) * K + k;
      if (k + 8 <= K && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
        *reinterpret_cast<uint2*>(dst) = out;
      } else {
        const uint8_t* b = reinterpret_cast<const uint8_t*>(&out);
        for (int i = 0; i < 8 && k + i < K; ++i) dst[i] = b[i];
      }
    }
  }
  if (!qt) return;
  __syncthreads();
  // transposed orientation: thread (tr, tc) writes 8 consecutive n for one k
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const int kk = p * 16 + tr;  // k within the tile
    const int k = kb * 128 + kk, n = nb * 128 + tc;
    if (k < K && n < N) {
      __align__(8) uint8_t b[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) b[i] = tile[tc + i][kk];
      uint8_t* dst = qt + ((long long)g * K + k) * N + n;
      if (n + 8 <= N && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0)) {
        *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(b);
      } else {
        for (int i = 0; i < 8 && n + i < N; ++i) dst[i] = b[i];
      }
    }
  }
}

}  // namespace pt

// x [*, K] bf16 (row pitch ldx elements) -> q [R, K] e4m3 + scales [ceil(K/128), ld_s].
// idx (optional, int32[R]) gathers rows of x: source row = idx[r] / div, negative = zero row;
// n_rows_dev (optional) is a device-side row count <= R.
PT_API int pt_quant_rows(const void* x, long long ldx, const int* idx, int div, const int* n_rows_dev, int R, int K,
                         void* q, float* s, long long ld_s, void* stream) {
  if (R <= 0 || K <= 0) return 0;
  if (K % 8 != 0) return -2;
  long long segs = (long long)R * ((K + 127) / 128);
  long long blocks = (segs + 15) / 16;
  int grid = (int)(blocks < (long long)pt::sm_count() * 16 ? blocks : (long long)pt::sm_count() * 16);
  pt::quant_rows_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, idx, div, n_rows_dev, R, K, reinterpret_cast<uint8_t*>(q), s, ld_s);
  return (int)cudaGetLastError();
}

// w [G, N, K] bf16 -> q [G, N, K], qt [G, K, N] (optional) e4m3; s [G, nb, kb], st [G, kb, nb] (optional).
PT_API int pt_quant_blocks(const void* w, int G, int N, int K, void* q, void* qt, float* s, float* st, void* stream) {
  if (G <= 0 || N <= 0 || K <= 0) return 0;
  dim3 grid((K + 127) / 128, (N + 127) / 128, G);
  pt::quant_block_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(w), N, K, reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(qt), s, st);
  return (int)cudaGetLastError();
}
