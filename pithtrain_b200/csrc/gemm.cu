// bf16 GEMM family for sm_100a: dense, M-grouped (expert forward / dgrad) and K-grouped (expert
// wgrad) in one persistent, warp-specialised kernel.
//
//   warp 0      TMA producer   : cp.async.bulk.tensor (no multicast) -> 128B-swizzled smem ring
//   warp 1      MMA issuer     : tcgen05.mma.cta_group::1.kind::f16, fp32 accumulators in TMEM,
//                                two accumulator buffers so the epilogue overlaps the next tile
//   warps 2..5  epilogue       : tcgen05.ld -> bf16/fp32 -> global (direct, optional accumulate,
//                                row-masked for ragged groups) or swizzled smem -> TMA store
//
// Operand layouts are chosen per operand: "K-major" (reduction dim contiguous: x[M,K], W[N,K]) or
// "MN-major" (reduction dim strided: W[N,K] used as the B of a dgrad, dy[M,N]/x[M,K] in a wgrad),
// so forward, dgrad and wgrad all read the tensors as they sit in memory — no transposes.
//
// Group boundaries come from a device-side offsets array, so no host synchronisation is needed to
// size anything: the grid is persistent and every CTA walks the same deterministic tile list.
// The role of the reference's DeepGEMM / F.grouped_mm calls
// (pithtrain/operators/grouped_linear.py:37-47,147,193,205-216, pithtrain/operators/linear.py:44-83).
#include "host_common.h"
#include "ptx.cuh"

namespace pt {

constexpr int BM = 128;
constexpr int BK = 64;  // bf16 elements per k-block = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;  // 16 KB
constexpr int EPI_WARPS = 4;

enum GemmMode : int { GEMM_DENSE = 0, GEMM_MGROUP = 1, GEMM_KGROUP = 2 };

struct GemmArgs {
  int M, N, K;  // dense: D[M,N], reduction K. mgroup: M = row capacity. kgroup: D_g[M,N], K from offs
  int mode;
  int num_groups;
  const int* offs;      // [num_groups + 1] row offsets (device memory)
  const int* offs2;     // kgroup only, optional: offsets of a second (A, B) operand pair whose rows are reduced into
                        // the same outputs in the same launch (two micro-batches share one pass over the gradient)
  int b_group_rows;     // rows of the B tensor map that belong to one group
  void* D;
  long long ldd;
  long long d_group_stride;  // kgroup: elements between consecutive group outputs
  int out_fp32;
  int accumulate;
  int use_tma_store;
  int epi;  // 0 staged coalesced rows, 1 direct per-thread rows, 2 TMA reduce-add when accumulating (else direct)
  int* err;
  // A-operand row gather (K-major A only): tile row r reads source row a_idx[r] / a_idx_div, a negative
  // index (or r >= a_idx_len) reads zeros. Replaces a separate gather pass over the activations.
  const int* a_idx;
  int a_idx_div;
  long long a_idx_len;
};

struct TileInfo {
  int am, ak;  // A tile origin: M coordinate, K coordinate base
  int bn, bk;  // B tile origin: N coordinate, K coordinate base
  int num_kb, last_steps;
  int k2, num_kb2, last_steps2;  // second operand pair of a kgroup launch: K base, k-blocks (0 = none), last block's steps
  int row0, row_end, col0;
  long long d_off;
};

template <int BN>
struct Scheduler {
  const GemmArgs& a;
  int t, stride;
  int m_tiles, n_tiles;
  int g, g_base;  // grouped modes: current group and the linear index of its first tile
  __device__ Scheduler(const GemmArgs& args) : a(args), t(blockIdx.x), stride(gridDim.x), g(0), g_base(0) {
    n_tiles = (a.N + BN - 1) / BN;
    m_tiles = (a.M + BM - 1) / BM;
  }
  __device__ bool next(TileInfo& ti) {
    if (a.mode == GEMM_DENSE) {
      if (t >= m_tiles * n_tiles) return false;
      // 8-row supergroups: concurrently running CTAs share A rows and B columns in L2.
      const int GROUP = 8;
      int per = GROUP * n_tiles;
      int gid = t / per, first_m = gid * GROUP;
      int gsz = min(m_tiles - first_m, GROUP);
      int local = t - gid * per;
      int mt = first_m + local % gsz, nt = local / gsz;
      ti.am = mt * BM; ti.ak = 0; ti.bn = nt * BN; ti.bk = 0;
      ti.num_kb = (a.K + BK - 1) / BK; ti.last_steps = BK / UMMA_K;
      ti.k2 = 0; ti.num_kb2 = 0; ti.last_steps2 = 0;
      ti.row0 = mt * BM; ti.row_end = a.M; ti.col0 = nt * BN; ti.d_off = 0;
      t += stride;
      return true;
    }
    while (g < a.num_groups) {
      int r0 = a.offs[g], r1 = a.offs[g + 1];
      int rows = r1 - r0;
      int q0 = 0, rows2 = 0;
      if (a.mode == GEMM_KGROUP && a.offs2) { q0 = a.offs2[g]; rows2 = a.offs2[g + 1] - q0; }
      int tiles;
      if (a.mode == GEMM_MGROUP) tiles = ((rows + BM - 1) / BM) * n_tiles;
      else tiles = (rows + rows2) > 0 ? m_tiles * n_tiles : 0;
      if (t < g_base + tiles) {
        int local = t - g_base;
        int mt = local / n_tiles, nt = local - mt * n_tiles;
        if (a.mode == GEMM_MGROUP) {
          ti.am = r0 + mt * BM; ti.ak = 0;
          ti.bn = nt * BN; ti.bk = 0;
          // B origin carries the group: K-major B adds rows to N, MN-major B adds rows to K.
          ti.bn += 0; ti.bk += 0;
          ti.num_kb = (a.K + BK - 1) / BK; ti.last_steps = BK / UMMA_K;
          ti.k2 = 0; ti.num_kb2 = 0; ti.last_steps2 = 0;
          ti.row0 = r0 + mt * BM; ti.row_end = r1; ti.col0 = nt * BN; ti.d_off = 0;
          ti.d_off = (long long)g;  // reused below as group index
        } else {
          ti.am = mt * BM; ti.ak = r0;
          ti.bn = nt * BN; ti.bk = r0;
          ti.num_kb = (rows + BK - 1) / BK;
          int rem = rows - (ti.num_kb - 1) * BK;
          ti.last_steps = (rem + UMMA_K - 1) / UMMA_K;
          ti.k2 = q0;
          ti.num_kb2 = (rows2 + BK - 1) / BK;
          int rem2 = rows2 - (ti.num_kb2 - 1) * BK;
          ti.last_steps2 = (rem2 + UMMA_K - 1) / UMMA_K;
          ti.row0 = mt * BM; ti.row_end = a.M; ti.col0 = nt * BN;
          ti.d_off = (long long)g;
        }
        t += stride;
        return true;
      }
      g_base += tiles;
      ++g;
    }
    return false;
  }
};

// DEEP_EPI trades operand ring depth for epilogue staging: the TMA reduce-add (a read-modify-write in L2) has a
// long latency, and with two 4 KB slabs per warp only 32 KB per SM are in flight; six slabs per warp keep the
// gradient accumulation of the short-K expert weight-gradient tiles fed.
template <int BN, bool A_MN, bool B_MN, bool A_GATHER, bool DEEP_EPI>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmA2,
                 const __grid_constant__ CUtensorMap tmB2, const GemmArgs args) {
  constexpr int B_TILE_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  constexpr int STAGES = DEEP_EPI ? 3 : ((BN == 256) ? 4 : 6);
  constexpr int NSTG = DEEP_EPI ? ((BN == 256) ? 5 : 6) : 2;  // staging slabs per epilogue warp
  constexpr int STAGING = EPI_WARPS * NSTG * 4096;
  constexpr uint32_t IDESC = make_idesc(1, 1, BM, BN, A_MN, B_MN);
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: power of two

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + STAGING);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (args.use_tma_store || args.epi == 2) tma_prefetch_desc(&tmD);
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
    // ------------------------------------------------------------------ TMA producer
    if (A_GATHER) {
      // every lane gathers four rows of the A tile per k-block (32 x 4 = 128 rows); lane 0 also
      // owns the barrier bookkeeping and the B tile
      Scheduler<BN> sch(args);
      TileInfo ti;
      uint32_t it = 0;
      bool ok = true;
      while (ok && sch.next(ti)) {
        int grp = (args.mode == GEMM_DENSE) ? 0 : (int)ti.d_off;
        int bn = ti.bn, bk = ti.bk;
        if (args.mode == GEMM_MGROUP) {
          if (B_MN) bk += grp * args.b_group_rows; else bn += grp * args.b_group_rows;
        }
        int r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          long long row = (long long)ti.am + 4 * lane + j;
          int v = (row < args.a_idx_len && row < ti.row_end) ? args.a_idx[row] : -1;
          r[j] = v >= 0 ? v / args.a_idx_div : -1;
        }
        for (int kb = 0; kb < ti.num_kb; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          int good = 1;
          if (lane == 0) good = mbar_wait_bounded(&empty[s], ph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER) ? 1 : 0;
          good = __shfl_sync(0xffffffffu, good, 0);
          if (!good) { ok = false; break; }
          if (lane == 0) mbar_expect_tx(&full[s], STAGE_BYTES);
          __syncwarp();
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          int kk = kb * BK;
          tma_gather4_2d(sa + lane * 512, &tmA, &full[s], ti.ak + kk, r[0], r[1], r[2], r[3]);
          if (lane == 0) {
            if (!B_MN) {
              tma_load_2d(sb, &tmB, &full[s], bk + kk, bn);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (BK * 128), &tmB, &full[s], bn + 64 * j, bk + kk);
            }
          }
        }
      }
      if (lane == 0 && *abort_flag) {
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
    } else if (lane == 0) {
      Scheduler<BN> sch(args);
      TileInfo ti;
      uint32_t it = 0;
      bool ok = true;
      while (ok && sch.next(ti)) {
        int grp = (args.mode == GEMM_DENSE) ? 0 : (int)ti.d_off;
        int bn = ti.bn, bk = ti.bk;
        if (args.mode == GEMM_MGROUP) {
          if (B_MN) bk += grp * args.b_group_rows; else bn += grp * args.b_group_rows;
        }
        const int total_kb = ti.num_kb + ti.num_kb2;
        for (int kb = 0; kb < total_kb; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait_bounded(&empty[s], ph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
          if (!ok) break;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          // the second operand pair of a kgroup launch continues the reduction of the same tile
          const bool second = kb >= ti.num_kb;
          const CUtensorMap* mA = second ? &tmA2 : &tmA;
          const CUtensorMap* mB = second ? &tmB2 : &tmB;
          const int ka = second ? ti.k2 + (kb - ti.num_kb) * BK : ti.ak + kb * BK;
          const int kbB = second ? ti.k2 + (kb - ti.num_kb) * BK : bk + kb * BK;
          if (!A_MN) {
            tma_load_2d(sa, mA, &full[s], ka, ti.am);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), mA, &full[s], ti.am + 64 * j, ka);
          }
          if (!B_MN) {
            tma_load_2d(sb, mB, &full[s], kbB, bn);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), mB, &full[s], bn + 64 * j, kbB);
          }
        }
      }
      if (*abort_flag) {
        // Gave up somewhere: let the copies already in flight land before the CTA retires.
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
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      Scheduler<BN> sch(args);
      TileInfo ti;
      uint32_t it = 0, tc = 0;
      bool ok = true;
      while (ok && sch.next(ti)) {
        int acc = tc & 1;
        uint32_t aph = (tc >> 1) & 1;
        ok = mbar_wait_bounded(&tmem_empty[acc], aph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        uint32_t d_tmem = tmem_base + acc * BN;
        const int total_kb = ti.num_kb + ti.num_kb2;
        for (int kb = 0; kb < total_kb; ++kb, ++it) {
          int s = it % STAGES;
          uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait_bounded(&full[s], ph, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          uint32_t b_addr = a_addr + A_TILE_BYTES;
          int steps = (kb == ti.num_kb - 1) ? ti.last_steps : (kb == total_kb - 1 && ti.num_kb2 > 0) ? ti.last_steps2 : (BK / UMMA_K);
          for (int k = 0; k < steps; ++k) {
            uint64_t ad = A_MN ? make_smem_desc_sw128(a_addr + k * 2048, BK * 128, 1024)
                               : make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            uint64_t bd = B_MN ? make_smem_desc_sw128(b_addr + k * 2048, BK * 128, 1024)
                               : make_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            umma_f16(d_tmem, ad, bd, IDESC, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // frees the smem stage once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        ++tc;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    Scheduler<BN> sch(args);
    TileInfo ti;
    uint32_t tc = 0;
    bool used_tma = false;
    uint32_t slab = 0;  // rotation through the staging slabs of this warp (TMA reduce epilogue)
    while (sch.next(ti)) {
      int acc = tc & 1;
      uint32_t aph = (tc >> 1) & 1;
      if (!mbar_wait_bounded(&tmem_full[acc], aph, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int row = ti.row0 + q * 32 + lane;
      const bool rvalid = row < ti.row_end;
      long long d_off = 0;
      if (args.mode == GEMM_KGROUP) d_off = ti.d_off * args.d_group_stride;
      const bool full_tile = (args.mode == GEMM_DENSE) || (ti.row0 + BM <= ti.row_end);
      if (args.use_tma_store && full_tile && !args.out_fp32 && !args.accumulate && args.mode != GEMM_KGROUP) {
        used_tma = true;
#pragma unroll 1
        for (int cc = 0; cc < BN / 64; ++cc) {
          if (ti.col0 + cc * 64 >= args.N) break;
          uint8_t* st = staging + (q * NSTG + (cc & 1)) * 4096;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + cc * 64, r0);
          tmem_ld_32x32(taddr + cc * 64 + 32, r1);
          tmem_ld_wait();
          uint8_t* rowp = st + lane * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
            v.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
            v.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
            v.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = v;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
            v.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
            v.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
            v.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
            *reinterpret_cast<uint4*>(rowp + (((j + 4) ^ (lane & 7)) << 4)) = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmD, st, ti.col0 + cc * 64, ti.row0 + q * 32);
            tma_store_commit();
          }
        }
      } else if (args.epi == 2 && args.accumulate && (args.mode != GEMM_MGROUP || full_tile)) {
        // ---- TMA reduce-add: stage a 32x(128 B) slab per warp, let the copy engine do D += slab
        used_tma = true;
        const int cols_per = args.out_fp32 ? 32 : 64;
#pragma unroll 1
        for (int cc = 0; cc * cols_per < BN; ++cc) {
          if (ti.col0 + cc * cols_per >= args.N) break;
          uint8_t* st = staging + (q * NSTG + (slab % NSTG)) * 4096;
          ++slab;
          if (lane == 0) tma_store_wait_read<NSTG - 1>();
          __syncwarp();
          uint8_t* rowp = st + lane * 128;
          if (args.out_fp32) {
            uint32_t r0[32];
            tmem_ld_32x32(taddr + cc * 32, r0);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(r0[4 * j], r0[4 * j + 1], r0[4 * j + 2], r0[4 * j + 3]);
          } else {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(taddr + cc * 64, r0);
            tmem_ld_32x32(taddr + cc * 64 + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v, w;
              v.x = pack_bf16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
              w.x = pack_bf16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
              w.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
              w.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
              w.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
              *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = v;
              *reinterpret_cast<uint4*>(rowp + (((j + 4) ^ (lane & 7)) << 4)) = w;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (args.mode == GEMM_KGROUP)
              tma_reduce_add_3d(&tmD, st, ti.col0 + cc * cols_per, ti.row0 + q * 32, (int)ti.d_off);
            else
              tma_reduce_add_2d(&tmD, st, ti.col0 + cc * cols_per, ti.row0 + q * 32);
            tma_store_commit();
          }
        }
      } else if (args.epi != 0) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = ti.col0 + c * 32;
          if (col >= args.N) break;  // uniform across the warp
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (rvalid) {
            if (args.out_fp32) {
              float* p = reinterpret_cast<float*>(args.D) + d_off + (long long)row * args.ldd + col;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (col + 4 * i < args.N) {
                  float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                         __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                  if (args.accumulate) {
                    float4 o = *reinterpret_cast<const float4*>(p + 4 * i);
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                  }
                  *reinterpret_cast<float4*>(p + 4 * i) = v;
                }
              }
            } else {
              __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(args.D) + d_off + (long long)row * args.ldd + col;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (col + 8 * i < args.N) {
                  float f[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * i + e]);
                  if (args.accumulate) {
                    uint4 o = *reinterpret_cast<const uint4*>(p + 8 * i);
                    float2 a0 = unpack_bf16x2(o.x), a1 = unpack_bf16x2(o.y), a2 = unpack_bf16x2(o.z), a3 = unpack_bf16x2(o.w);
                    f[0] += a0.x; f[1] += a0.y; f[2] += a1.x; f[3] += a1.y;
                    f[4] += a2.x; f[5] += a2.y; f[6] += a3.x; f[7] += a3.y;
                  }
                  uint4 v;
                  v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
                  v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
                  *reinterpret_cast<uint4*>(p + 8 * i) = v;
                }
              }
            }
          }
        }
      } else {
        // ---- staged: registers -> swizzled smem slab -> coalesced 128-byte row segments in global
        // (read-modify-write when accumulating). Handles ragged rows/columns and both output dtypes.
        uint8_t* st = staging + q * NSTG * 4096;
        const int cols_per = args.out_fp32 ? 32 : 64;
        const int sub_row = lane >> 3, chunk = lane & 7;
#pragma unroll 1
        for (int cc = 0; cc * cols_per < BN; ++cc) {
          const int col_base = ti.col0 + cc * cols_per;
          if (col_base >= args.N) break;
          uint8_t* rowp = st + lane * 128;
          __syncwarp();
          if (args.out_fp32) {
            uint32_t r0[32];
            tmem_ld_32x32(taddr + cc * 32, r0);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(r0[4 * j], r0[4 * j + 1], r0[4 * j + 2], r0[4 * j + 3]);
          } else {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(taddr + cc * 64, r0);
            tmem_ld_32x32(taddr + cc * 64 + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v, w;
              v.x = pack_bf16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
              w.x = pack_bf16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
              w.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
              w.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
              w.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
              *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = v;
              *reinterpret_cast<uint4*>(rowp + (((j + 4) ^ (lane & 7)) << 4)) = w;
            }
          }
          __syncwarp();
          const int elems_per_chunk = args.out_fp32 ? 4 : 8;
          const int col = col_base + chunk * elems_per_chunk;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rloc = it * 4 + sub_row;
            const int grow = ti.row0 + q * 32 + rloc;
            if (grow < ti.row_end && col < args.N) {
              uint4 v = *reinterpret_cast<const uint4*>(st + rloc * 128 + ((chunk ^ (rloc & 7)) << 4));
              if (args.out_fp32) {
                float* p = reinterpret_cast<float*>(args.D) + d_off + (long long)grow * args.ldd + col;
                if (args.accumulate) {
                  float4 o = *reinterpret_cast<const float4*>(p);
                  v.x = __float_as_uint(__uint_as_float(v.x) + o.x); v.y = __float_as_uint(__uint_as_float(v.y) + o.y);
                  v.z = __float_as_uint(__uint_as_float(v.z) + o.z); v.w = __float_as_uint(__uint_as_float(v.w) + o.w);
                }
                *reinterpret_cast<uint4*>(p) = v;
              } else {
                __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(args.D) + d_off + (long long)grow * args.ldd + col;
                if (args.accumulate) {
                  uint4 o = *reinterpret_cast<const uint4*>(p);
                  float2 a0 = unpack_bf16x2(v.x), a1 = unpack_bf16x2(v.y), a2 = unpack_bf16x2(v.z), a3 = unpack_bf16x2(v.w);
                  float2 b0 = unpack_bf16x2(o.x), b1 = unpack_bf16x2(o.y), b2 = unpack_bf16x2(o.z), b3 = unpack_bf16x2(o.w);
                  v.x = pack_bf16x2(a0.x + b0.x, a0.y + b0.y); v.y = pack_bf16x2(a1.x + b1.x, a1.y + b1.y);
                  v.z = pack_bf16x2(a2.x + b2.x, a2.y + b2.y); v.w = pack_bf16x2(a3.x + b3.x, a3.y + b3.y);
                }
                *reinterpret_cast<uint4*>(p) = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      ++tc;
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

template <int BN, bool DEEP_EPI>
constexpr int gemm_smem_bytes() {
  return (DEEP_EPI ? 3 : ((BN == 256) ? 4 : 6)) * (A_TILE_BYTES + BN * BK * 2) +
         EPI_WARPS * (DEEP_EPI ? ((BN == 256) ? 5 : 6) : 2) * 4096 + 256 + 1024;
}

template <int BN, bool A_MN, bool B_MN, bool A_GATHER = false, bool DEEP_EPI = false>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD,
                const GemmArgs& args, int grid, cudaStream_t stream, const CUtensorMap* tmA2 = nullptr,
                const CUtensorMap* tmB2 = nullptr) {
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, A_GATHER, DEEP_EPI>;
  constexpr int smem = gemm_smem_bytes<BN, DEEP_EPI>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, 192, smem, stream>>>(tmA, tmB, tmD, tmA2 ? *tmA2 : tmA, tmB2 ? *tmB2 : tmB, args);
  return (int)cudaGetLastError();
}

}  // namespace pt

// D = A * B (+ D), bf16 inputs, fp32 accumulation on the tensor cores.
//   mode 0 dense   : A is [M,K] (K-major) or [K,M] (MN-major); B is [N,K] or [K,N]; D [M,N].
//   mode 1 mgroup  : rows of A/D are split into groups by `offs`; group g uses B rows
//                    [g*b_group_rows, (g+1)*b_group_rows) (added to N for K-major B, to K for MN-major B).
//   mode 2 kgroup  : group g reduces over rows [offs[g], offs[g+1]) of A [R,M] and B [R,N] (both
//                    MN-major) into D + g*d_group_stride (always accumulates when accumulate=1;
//                    groups with zero rows are left untouched). Group sizes must be multiples of 16.
// a_rows/a_cols/lda etc. describe each operand as the row-major matrix it is in memory.
// a_idx (optional, K-major A only): row r of the GEMM's A is source row a_idx[r] / a_idx_div of the
// tensor described by a_rows/a_cols/lda (negative index or r >= a_idx_len: a zero row), fetched with
// TMA gather4 straight into the swizzled operand tile.
// Returns 0 on success.
PT_API int pt_gemm_bf16(const void* A, const void* B, void* D, int mode, int M, int N, int K,
                        int a_mn, int b_mn, long long a_rows, long long a_cols, long long lda,
                        long long b_rows, long long b_cols, long long ldb, long long d_rows,
                        long long ldd, const int* offs, int num_groups, int b_group_rows,
                        long long d_group_stride, int out_fp32, int accumulate,
                        int use_tma_store, int epi, int bn, int max_ctas, const int* a_idx, int a_idx_div,
                        long long a_idx_len, void* stream_) {
  using namespace pt;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (mode == GEMM_DENSE && K <= 0) return 0;
  if (bn != 128 && bn != 256) bn = (N >= 256) ? 256 : 128;
  CUtensorMap tmA, tmB, tmD;
  int rc;
  const bool gather = a_idx != nullptr;
  if (gather && a_mn) return -3;  // row gather is implemented for K-major A only
  if (gather) rc = encode_tmap_2d(&tmA, A, TM_BF16, a_rows, a_cols, lda, 1, BK, TM_SW_128);
  else if (!a_mn) rc = encode_tmap_2d(&tmA, A, TM_BF16, a_rows, a_cols, lda, BM, BK, TM_SW_128);
  else rc = encode_tmap_2d(&tmA, A, TM_BF16, a_rows, a_cols, lda, BK, 64, TM_SW_128);
  if (rc) return 1000 + rc;
  if (!b_mn) rc = encode_tmap_2d(&tmB, B, TM_BF16, b_rows, b_cols, ldb, bn, BK, TM_SW_128);
  else rc = encode_tmap_2d(&tmB, B, TM_BF16, b_rows, b_cols, ldb, BK, 64, TM_SW_128);
  if (rc) return 2000 + rc;
  bool tma_store_ok = use_tma_store && !out_fp32 && !accumulate && mode != GEMM_KGROUP && (N % 8 == 0);
  bool tma_reduce = (epi == 2) && accumulate && (N % 8 == 0);
  if (tma_store_ok) {
    rc = encode_tmap_2d(&tmD, D, TM_BF16, d_rows, N, ldd, 32, 64, TM_SW_128);
    if (rc) return 3000 + rc;
  } else if (tma_reduce) {
    TmDtype dt = out_fp32 ? TM_F32 : TM_BF16;
    uint32_t box_cols = out_fp32 ? 32 : 64;
    if (mode == GEMM_KGROUP)
      rc = encode_tmap_3d(&tmD, D, dt, num_groups, M, N, ldd, d_group_stride, 1, 32, box_cols, TM_SW_128);
    else
      rc = encode_tmap_2d(&tmD, D, dt, d_rows, N, ldd, 32, box_cols, TM_SW_128);
    if (rc) return 3000 + rc;
  } else {
    tmD = tmA;
    if (epi == 2) epi = 1;
  }
  GemmArgs args;
  args.M = M; args.N = N; args.K = K; args.mode = mode; args.num_groups = num_groups;
  args.offs = offs; args.offs2 = nullptr; args.b_group_rows = b_group_rows; args.D = D; args.ldd = ldd;
  args.d_group_stride = d_group_stride; args.out_fp32 = out_fp32; args.accumulate = accumulate;
  args.use_tma_store = tma_store_ok ? 1 : 0;
  args.epi = epi;
  args.err = device_status_word();
  args.a_idx = a_idx; args.a_idx_div = a_idx_div > 0 ? a_idx_div : 1; args.a_idx_len = a_idx_len;

  int sms = sm_count();
  int grid = sms;
  if (mode == GEMM_DENSE) {
    long long tiles = (long long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    if (tiles < grid) grid = (int)tiles;
  }
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid <= 0) return 0;

  if (gather) {
    if (bn == 256) return b_mn ? launch_gemm<256, false, true, true>(tmA, tmB, tmD, args, grid, stream)
                               : launch_gemm<256, false, false, true>(tmA, tmB, tmD, args, grid, stream);
    return b_mn ? launch_gemm<128, false, true, true>(tmA, tmB, tmD, args, grid, stream)
                : launch_gemm<128, false, false, true>(tmA, tmB, tmD, args, grid, stream);
  }
  if (mode == GEMM_KGROUP && tma_reduce && a_mn && b_mn) {
    return bn == 256 ? launch_gemm<256, true, true, false, true>(tmA, tmB, tmD, args, grid, stream)
                     : launch_gemm<128, true, true, false, true>(tmA, tmB, tmD, args, grid, stream);
  }
  int key = (bn == 256 ? 4 : 0) | (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  switch (key) {
    case 0: return launch_gemm<128, false, false>(tmA, tmB, tmD, args, grid, stream);
    case 1: return launch_gemm<128, false, true>(tmA, tmB, tmD, args, grid, stream);
    case 2: return launch_gemm<128, true, false>(tmA, tmB, tmD, args, grid, stream);
    case 3: return launch_gemm<128, true, true>(tmA, tmB, tmD, args, grid, stream);
    case 4: return launch_gemm<256, false, false>(tmA, tmB, tmD, args, grid, stream);
    case 5: return launch_gemm<256, false, true>(tmA, tmB, tmD, args, grid, stream);
    case 6: return launch_gemm<256, true, false>(tmA, tmB, tmD, args, grid, stream);
    case 7: return launch_gemm<256, true, true>(tmA, tmB, tmD, args, grid, stream);
  }
  return -1;
}

// Expert weight gradients of two micro-batches in one launch: for every group g,
//   D_g += A1[offs1[g]:offs1[g+1]]^T B1[...] + A2[offs2[g]:offs2[g+1]]^T B2[...]
// (A* [R*, M], B* [R*, N] bf16 row-major, read MN-major; D [G, M, N] bf16 or fp32, accumulated with TMA reduce-add).
// One pass over the gradient buffer instead of two: the launch is bound by that read-modify-write, not by its FLOPs.
// Group sizes must be multiples of 16 in both operand pairs.
PT_API int pt_gemm_bf16_kgroup2(const void* A1, const void* B1, const int* offs1, long long rows1, const void* A2,
                                const void* B2, const int* offs2, long long rows2, void* D, int M, int N, long long lda,
                                long long ldb, long long ldd, long long d_group_stride, int num_groups, int out_fp32,
                                void* stream_) {
  using namespace pt;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || num_groups <= 0) return 0;
  if (N % 8 != 0 || rows1 <= 0 || rows2 <= 0) return -2;
  const int bn = (N >= 256) ? 256 : 128;
  CUtensorMap tmA, tmB, tmA2, tmB2, tmD;
  if (encode_tmap_2d(&tmA, A1, TM_BF16, rows1, M, lda, BK, 64, TM_SW_128)) return 1001;
  if (encode_tmap_2d(&tmB, B1, TM_BF16, rows1, N, ldb, BK, 64, TM_SW_128)) return 2001;
  if (encode_tmap_2d(&tmA2, A2, TM_BF16, rows2, M, lda, BK, 64, TM_SW_128)) return 1002;
  if (encode_tmap_2d(&tmB2, B2, TM_BF16, rows2, N, ldb, BK, 64, TM_SW_128)) return 2002;
  if (encode_tmap_3d(&tmD, D, out_fp32 ? TM_F32 : TM_BF16, num_groups, M, N, ldd, d_group_stride, 1, 32, out_fp32 ? 32 : 64,
                     TM_SW_128))
    return 3001;
  GemmArgs args;
  args.M = M; args.N = N; args.K = 0; args.mode = GEMM_KGROUP; args.num_groups = num_groups;
  args.offs = offs1; args.offs2 = offs2; args.b_group_rows = 0; args.D = D; args.ldd = ldd;
  args.d_group_stride = d_group_stride; args.out_fp32 = out_fp32; args.accumulate = 1;
  args.use_tma_store = 0;
  args.epi = 2;
  args.err = device_status_word();
  args.a_idx = nullptr; args.a_idx_div = 1; args.a_idx_len = 0;
  const int grid = sm_count();
  return bn == 256 ? launch_gemm<256, true, true, false, true>(tmA, tmB, tmD, args, grid, stream, &tmA2, &tmB2)
                   : launch_gemm<128, true, true, false, true>(tmA, tmB, tmD, args, grid, stream, &tmA2, &tmB2);
}
