// Block-scaled FP8 (e4m3) GEMM for sm_100a: D[M,N] (bf16) = (A .* sa) * (B .* sb)^T.
//
//   A [M,K] e4m3, one power-of-two scale per 1x128 row segment   (activations / output gradients)
//   B [N,K] e4m3, one power-of-two scale per 128x128 tile        (weights, either orientation)
//
// The tensor cores run tcgen05.mma.kind::f8f6f4 over one 128-wide k-block at a time into one of
// two TMEM buffers; the eight epilogue warps pull each finished k-block partial out of TMEM and
// fold it into fp32 register accumulators with that block's scale (sa[row,kb] * sb[tile,kb]) while
// the tensor cores already work on the next k-block in the other buffer — two-level accumulation
// with the promotion running concurrently with the MMAs instead of stalling them.
//
//   warp 0      TMA producer   : A (128 rows) and B (256 rows) k-blocks of 128 bytes, 128B swizzle, into a ring
//   warp 1      MMA issuer     : 4 x (M128 N256 K32) per k-block, commit -> smem stage free, TMEM full
//   warps 2..9  promotion + epilogue: tcgen05.ld, scaled FMA, bf16 store (TMA store or direct rows);
//               two warps per TMEM lane quarter, each owning one 128-column half of the tile (= one
//               128-wide weight scale block)
//
// Modes: dense, and M-grouped (expert GEMMs: rows grouped by a device-side offsets array, group g
// uses weight rows [g*b_group_rows, ...)). Takes the role of DeepGEMM's fp8_gemm_nt and
// m_grouped_fp8_gemm_nt_contiguous in the reference (pithtrain/operators/linear.py:40-83,
// pithtrain/operators/grouped_linear.py:88-101,147,193).
#include "host_common.h"
#include "ptx.cuh"

namespace pt {
namespace f8 {

constexpr int BM = 128, BN = 256, BK = 128;  // BK bytes = one 128-byte swizzle row = one scale block
constexpr int UMMA_K = 32;
constexpr int TILE_BYTES = BM * BK;    // A: 16 KB per stage
constexpr int B_TILE_BYTES = BN * BK;  // B: 32 KB per stage
constexpr int STAGE_BYTES = TILE_BYTES + B_TILE_BYTES;
constexpr int STAGES = 4;
constexpr int EPI_WARPS = 8;  // two per TMEM lane quarter: each folds one 64-column half of the tile
constexpr int STAGING_BYTES = EPI_WARPS * 4096;
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int NBUF = 2;  // k-block accumulators in flight
constexpr uint32_t TMEM_COLS = NBUF * BN;  // 512: the whole tensor memory of the SM
constexpr uint32_t IDESC = make_idesc(0, 0, BM, BN, false, false);

struct Args {
  int M, N, K;
  int mode;  // 0 dense, 1 m-grouped
  int num_groups;
  const int* offs;
  int b_group_rows;
  const float* sa;  // [kblocks, ld_sa]
  long long ld_sa;
  const float* sb;  // [groups, nblocks, kblocks]
  __nv_bfloat16* D;
  long long ldd;
  int use_tma_store;
  int* err;
};

struct Tile {
  int am, bn, row0, row_end, col0, grp, nt;
};

struct Sched {
  const Args& a;
  int t, stride, m_tiles, n_tiles, g, g_base;
  __device__ Sched(const Args& args) : a(args), t(blockIdx.x), stride(gridDim.x), g(0), g_base(0) {
    n_tiles = (a.N + BN - 1) / BN;
    m_tiles = (a.M + BM - 1) / BM;
  }
  __device__ bool next(Tile& ti) {
    if (a.mode == 0) {
      if (t >= m_tiles * n_tiles) return false;
      const int GROUP = 8;
      int per = GROUP * n_tiles;
      int gid = t / per, first_m = gid * GROUP;
      int gsz = min(m_tiles - first_m, GROUP);
      int local = t - gid * per;
      int mt = first_m + local % gsz, nt = local / gsz;
      ti.am = mt * BM; ti.bn = nt * BN; ti.row0 = mt * BM; ti.row_end = a.M; ti.col0 = nt * BN;
      ti.grp = 0; ti.nt = nt;
      t += stride;
      return true;
    }
    while (g < a.num_groups) {
      int r0 = a.offs[g], r1 = a.offs[g + 1];
      int tiles = ((r1 - r0 + BM - 1) / BM) * n_tiles;
      if (t < g_base + tiles) {
        int local = t - g_base;
        int mt = local / n_tiles, nt = local - mt * n_tiles;
        ti.am = r0 + mt * BM; ti.bn = nt * BN + g * a.b_group_rows;
        ti.row0 = ti.am; ti.row_end = r1; ti.col0 = nt * BN; ti.grp = g; ti.nt = nt;
        t += stride;
        return true;
      }
      g_base += tiles;
      ++g;
    }
    return false;
  }
};

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmD, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + STAGING_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + NBUF;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_empty + NBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (args.K + BK - 1) / BK;
  const int last_steps = ((args.K - (num_kb - 1) * BK) + UMMA_K - 1) / UMMA_K;
  const int nblocks = (args.N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < NBUF; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (args.use_tma_store) tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    if (lane == 0) {
      Sched sch(args);
      Tile ti;
      uint32_t it = 0;
      bool ok = true;
      while (ok && sch.next(ti)) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait_bounded(&empty[s], ph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
          if (!ok) break;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          uint8_t* sa = smem + s * STAGE_BYTES;
          tma_load_2d(sa, &tmA, &full[s], kb * BK, ti.am);
          tma_load_2d(sa + TILE_BYTES, &tmB, &full[s], kb * BK, ti.bn);  // 256 rows x 128 bytes
        }
      }
      if (*abort_flag) {
        uint32_t n = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        for (uint32_t j = 0; j < n; ++j) {
          uint32_t jt = it - 1 - j;
          int s = jt % STAGES;
          uint32_t ph = (jt / STAGES) & 1;
          uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full[s], ph)) {
            if (globaltimer_ns() - t0 > 20000000ull) {
              if (args.err) atomicCAS(args.err, 0, PT_ERR_TIMEOUT_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      Sched sch(args);
      Tile ti;
      uint32_t it = 0;  // k-block counter: selects both the smem stage and the TMEM buffer
      bool ok = true;
      while (ok && sch.next(ti)) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          int buf = it % NBUF;
          uint32_t bph = (it / NBUF) & 1;
          ok = mbar_wait_bounded(&tmem_empty[buf], bph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait_bounded(&full[s], ph, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          uint32_t b_addr = a_addr + TILE_BYTES;
          uint32_t d_tmem = tmem_base + buf * BN;
          int steps = (kb == num_kb - 1) ? last_steps : (BK / UMMA_K);
          for (int k = 0; k < steps; ++k) {
            uint64_t ad = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            uint64_t bd = make_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            umma_f8(d_tmem, ad, bd, IDESC, k != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          umma_commit(&tmem_full[buf]);
        }
      }
    }
  } else {
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;  // which half (128 columns) of the tile this warp folds
    constexpr int HC = BN / 2;
    Sched sch(args);
    Tile ti;
    uint32_t it = 0;
    bool used_tma = false, ok = true;
    uint8_t* st = staging + (warp - 2) * 4096;
    while (ok && sch.next(ti)) {
      const int row = ti.row0 + q * 32 + lane;
      const bool rvalid = row < ti.row_end;
      const float* sa_p = args.sa + row;
      const int nb_idx = min(ti.nt * (BN / 128) + half, nblocks - 1);  // the 128-wide weight block of this half
      const float* sb_p = args.sb + ((long long)ti.grp * nblocks + nb_idx) * num_kb;
      float acc[HC];
#pragma unroll
      for (int i = 0; i < HC; ++i) acc[i] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int buf = it % NBUF;
        const uint32_t bph = (it / NBUF) & 1;
        const float sc = (rvalid ? sa_p[(long long)kb * args.ld_sa] : 0.f) * sb_p[kb];
        // one lane polls the barrier, the warp follows: 8 pollers per CTA instead of 256
        int good = 1;
        if (lane == 0) good = mbar_wait_bounded(&tmem_full[buf], bph, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        ok = good != 0;
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + half * HC;
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (c == HC / 32 - 1) {
            // the whole partial has left TMEM: hand the buffer back before the last arithmetic
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(__uint_as_float(r[j]), sc, acc[c * 32 + j]);
        }
      }
      if (!ok) break;
      const bool full_tile = (args.mode == 0) ? (ti.row0 + BM <= args.M) : (ti.row0 + BM <= ti.row_end);
      const int col0 = ti.col0 + half * HC;
      if (col0 >= args.N) continue;  // uniform across the warp
      if (args.use_tma_store && full_tile) {
        used_tma = true;
#pragma unroll
        for (int cc = 0; cc < HC / 64; ++cc) {
          if (col0 + cc * 64 < args.N) {
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
            uint8_t* rowp = st + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint4 v;
              v.x = pack_bf16x2(acc[cc * 64 + 8 * j + 0], acc[cc * 64 + 8 * j + 1]);
              v.y = pack_bf16x2(acc[cc * 64 + 8 * j + 2], acc[cc * 64 + 8 * j + 3]);
              v.z = pack_bf16x2(acc[cc * 64 + 8 * j + 4], acc[cc * 64 + 8 * j + 5]);
              v.w = pack_bf16x2(acc[cc * 64 + 8 * j + 6], acc[cc * 64 + 8 * j + 7]);
              *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmD, st, col0 + cc * 64, ti.row0 + q * 32);
              tma_store_commit();
            }
          }
        }
      } else if (rvalid) {
        __nv_bfloat16* p = args.D + (long long)row * args.ldd + col0;
#pragma unroll
        for (int i = 0; i < HC / 8; ++i) {
          if (col0 + 8 * i < args.N) {
            uint4 v;
            v.x = pack_bf16x2(acc[8 * i + 0], acc[8 * i + 1]);
            v.y = pack_bf16x2(acc[8 * i + 2], acc[8 * i + 3]);
            v.z = pack_bf16x2(acc[8 * i + 4], acc[8 * i + 5]);
            v.w = pack_bf16x2(acc[8 * i + 6], acc[8 * i + 7]);
            *reinterpret_cast<uint4*>(p + 8 * i) = v;
          }
        }
      }
    }
    if (used_tma && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 256 + 1024;

}  // namespace f8
}  // namespace pt

// D [*, N] bf16 = A [*, K] e4m3 (row scales sa [ceil(K/128), ld_sa]) times B [b_rows, K] e4m3 (tile
// scales sb [groups, ceil(N/128), ceil(K/128)]) transposed. mode 0 dense over M rows; mode 1 M-grouped:
// rows [offs[g], offs[g+1]) use B rows [g*b_group_rows, g*b_group_rows + N). K and N multiples of 16.
PT_API int pt_gemm_fp8(const void* A, const void* B, void* D, int mode, int M, int N, int K, long long a_rows,
                       long long b_rows, long long d_rows, long long ldd, const float* sa, long long ld_sa,
                       const float* sb, const int* offs, int num_groups, int b_group_rows, int use_tma_store,
                       int max_ctas, void* stream_) {
  using namespace pt;
  using namespace pt::f8;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 16 != 0 || N % 8 != 0) return -2;
  CUtensorMap tmA, tmB, tmD;
  int rc = encode_tmap_2d(&tmA, A, TM_U8, a_rows, K, K, BM, BK, TM_SW_128);
  if (rc) return 1000 + rc;
  rc = encode_tmap_2d(&tmB, B, TM_U8, b_rows, K, K, BN, BK, TM_SW_128);
  if (rc) return 2000 + rc;
  if (use_tma_store) {
    rc = encode_tmap_2d(&tmD, D, TM_BF16, d_rows, N, ldd, 32, 64, TM_SW_128);
    if (rc) return 3000 + rc;
  } else {
    tmD = tmA;
  }
  Args args;
  args.M = M; args.N = N; args.K = K; args.mode = mode; args.num_groups = num_groups; args.offs = offs;
  args.b_group_rows = b_group_rows; args.sa = sa; args.ld_sa = ld_sa; args.sb = sb;
  args.D = reinterpret_cast<__nv_bfloat16*>(D); args.ldd = ldd; args.use_tma_store = use_tma_store ? 1 : 0;
  args.err = device_status_word();
  int grid = sm_count();
  if (mode == 0) {
    long long tiles = (long long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    if (tiles < grid) grid = (int)tiles;
  }
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  gemm_fp8_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmD, args);
  return (int)cudaGetLastError();
}
