// Attention backward for sm_100a (tcgen05 / TMEM / TMA): dQ, dK, dV of bf16 attention with the masks of the forward
// kernel (causal or unmasked, per-row lower key bounds for sliding windows and packed documents, GQA), head dims 64
// and 128. Takes the role of the reference's FlashAttention-4 backward (pithtrain/operators/flash_attn_v4.py:29-45,
// :71-87). S and dP are recomputed from Q, K, V, dO and the forward's log-sum-exp; nothing of size S x S is stored.
//
//   pre  : delta[b,h,r] = sum_d dO*O (fp32) and lse2 = lse * log2(e); the fp32 accumulators are zeroed by the caller
//   main : grid = (Hq * B, key tiles). A CTA owns one 128-key tile of one query head (K, V tiles stay in shared memory)
//          and walks the query tiles i that can see it. Everything is computed transposed, so that a thread owns a
//          key row and the dK / dV accumulators (rows = keys) stay in TMEM for the whole walk:
//            S^T  = K Q_i^T              -> TMEM region R[n&1]
//            dP^T = V dO_i^T             -> TMEM region R[1-(n&1)]
//            P^T  = exp2(S^T*c - lse2)   -> packed bf16 over S^T in TMEM      (A operand of the dV MMA, from TMEM)
//            dS^T = P^T o (dP^T - delta) -> bf16 tile in shared memory        (A operand of dK and, read the other
//                                                                              way round, of dQ)
//            dV  += P^T dO_i    dK += dS^T Q_i    dQ_i = dS K -> TMEM region R[n&1] (free once dV has read P^T)
//          dQ_i leaves through registers and a swizzled staging tile as a TMA reduce-add into an fp32 accumulator.
//          The tensor core runs dP(n), dV(n), S(n+1), dK(n), dQ(n): the next S^T is issued as soon as dP^T has been
//          read, so the exponentials of step n+1 overlap the dK / dQ MMAs of step n.
//          warp 0 TMA producer | warps 1, 2 MMA issuers (S^T, dP^T | dV, dK, dQ) | warps 4..11 two compute warp groups
//          (64 query columns each) | warps 12..15 dQ reduction and the final dK / dV reduce-add (fp32, summed over the
//          heads of a GQA group). setmaxnreg moves registers from the first warp group to the others.
//   post : dq = bf16(acc * scale), dk = bf16(acc * scale), dv = bf16(acc).
//
// Every wait is bounded (mbar_wait_bounded); on a timeout the roles leave their loops, the CTA frees its TMEM and
// the status word carries the code.
#include <type_traits>

#include "host_common.h"
#include "ptx.cuh"

namespace pt {

constexpr int AB_SLAB = 128 * 64 * 2;  // one [128 x 64] bf16 swizzle slab: 16 KB
#ifndef AB_EXP_CHUNK
#define AB_EXP_CHUNK 32  // query columns per pass of the rolled exponential loop (32 or 16; measured 447 / 469 us)
#endif
#ifndef AB_POLY_MASK
// Which of every 8 exponentials take the polynomial on the FMA pipe (see exp2_poly). Measured (all five backward
// launches, 1 x 4096 x 32/4 heads x 128, causal): 0x00 554 us, 0x55 592 us, 0xB5 612 us, 0xFF 636 us: none is the default.
#define AB_POLY_MASK 0x00u
#endif

struct AttnBwdArgs {
  int B, Sq, Sk, Hq, Hkv;
  int causal, q_off;
  float scale_log2;
  const int* row_lo;    // optional [B*Sq]
  const float* lse2;    // [B, Hq, Sq] log2-domain log-sum-exp (+inf for rows that saw no key)
  const float* delta;   // [B, Hq, Sq]
  int* err;
};

template <int D>
struct AttnBwdCfg {
  static constexpr int T_BYTES = (D / 64) * AB_SLAB;          // one [128 x D] bf16 tile
  static constexpr int DS_BYTES = 2 * AB_SLAB;                // dS^T [128 keys x 128 queries] bf16
  static constexpr int STG_BYTES = 4 * 2 * 4096;              // 4 reduce warps x 2 staging tiles of [32 x 32] fp32
  static constexpr int STAT_BYTES = 2 * 1024;                  // two stages of lse2[128] | delta[128]
  static constexpr int BAR_BYTES = 256;
  // K, V, Q x2, dO, dS, staging, row statistics. No slack for re-aligning the base: the kernel checks that the dynamic
  // shared-memory window starts on a 1024-byte boundary (the swizzled tiles need it) and reports if it does not.
  static constexpr int SMEM = 5 * T_BYTES + DS_BYTES + STG_BYTES + STAT_BYTES + BAR_BYTES;
  static constexpr int THREADS = 16 * 32;
};

template <int D>
__global__ void __launch_bounds__(512, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                const __grid_constant__ CUtensorMap tmDV, const AttnBwdArgs args) {
  using Cfg = AttnBwdCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {  // uniform over the CTA
    if (threadIdx.x == 0 && args.err) atomicCAS(args.err, 0, PT_ERR_SMEM_ALIGN);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::T_BYTES;
  uint8_t* sQ = sV + Cfg::T_BYTES;           // two stages
  uint8_t* sDO = sQ + 2 * Cfg::T_BYTES;
  uint8_t* sDS = sDO + Cfg::T_BYTES;
  uint8_t* sStg = sDS + Cfg::DS_BYTES;
  uint8_t* sStat = sStg + Cfg::STG_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + Cfg::STAT_BYTES);
  uint64_t* kv_full = bars;        // 1
  uint64_t* q_full = bars + 1;     // 2
  uint64_t* q_empty = bars + 3;    // 2
  uint64_t* do_full = bars + 5;    // 1
  uint64_t* do_empty = bars + 6;   // 1
  uint64_t* s_full = bars + 7;     // MMA -> compute
  uint64_t* dp_full = bars + 8;    // MMA -> compute
  uint64_t* p_ready = bars + 9;    // compute (8 warps) -> MMA: P^T is in TMEM; steps alternate between this barrier and
                                   // p_ready2 (the compute warps reach the next step's arrival without any help from the
                                   // back issuer, so a single barrier could come round before that thread has looked)
  uint64_t* dp_read = bars + 10;   // compute (8 warps) -> MMA: dP^T has left TMEM
  uint64_t* ds_ready = bars + 11;  // compute (8 warps) -> MMA: dS^T is in shared memory
  uint64_t* dq_full = bars + 12;   // MMA -> reduce warps
  uint64_t* dq_read = bars + 13;   // reduce (4 warps) -> MMA: dQ has left TMEM
  uint64_t* all_done = bars + 14;  // MMA -> reduce warps: dK / dV complete
  uint64_t* dk_done = bars + 15;   // MMA -> compute: the dK product of a step has read dS^T (its tile may be rewritten)
  uint64_t* p_ready2 = bars + 16;  // odd steps' P^T barrier
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads and batch entries along x, key tiles along y: blocks start in linear order (x fastest), so under a causal
  // mask the key tiles with the most query tiles (the first ones) start first on every SM
  const int j = blockIdx.y, hq = blockIdx.x % args.Hq, b = blockIdx.x / args.Hq;
  const int hk = hq / (args.Hq / args.Hkv);
  const int nQ = (args.Sq + 127) / 128;
  const int row_base = b * args.Sq, kv_base = b * args.Sk;
  const int k_first = j * 128, k_last = min(j * 128 + 127, args.Sk - 1);

  // query tiles [i_lo, i_hi] that can see this key tile (hi and lo of a row are non-decreasing in the row index)
  int i_lo = 0, i_hi = nQ - 1;
  if (args.causal) {
    const int need = k_first - args.q_off - 127;  // last row of tile i: q_off + 128 i + 127 >= k_first
    i_lo = need > 0 ? (need + 127) / 128 : 0;
  }
  if (args.row_lo && i_lo <= i_hi) {
    // largest i with row_lo[first row of tile i] <= k_last
    int a = i_lo, z = i_hi;
    if (args.row_lo[row_base + a * 128] > k_last) {
      i_hi = i_lo - 1;
    } else {
      while (a < z) {
        const int mid = (a + z + 1) >> 1;
        if (args.row_lo[row_base + mid * 128] <= k_last) a = mid; else z = mid - 1;
      }
      i_hi = a;
    }
  }
  const int N = i_hi - i_lo + 1;
  if (N <= 0) return;  // uniform over the CTA: nothing allocated yet

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 2); }  // both issuers release
    mbar_init(do_full, 1); mbar_init(do_empty, 2);
    mbar_init(s_full, 1); mbar_init(dp_full, 1);
    mbar_init(p_ready, 8); mbar_init(p_ready2, 8); mbar_init(dp_read, 8); mbar_init(ds_ready, 8);
    mbar_init(dq_full, 1); mbar_init(dq_read, 4); mbar_init(all_done, 1); mbar_init(dk_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQ); tma_prefetch_desc(&tmDK); tma_prefetch_desc(&tmDV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const uint32_t tDK = tmem_base + 256, tDV = tmem_base + 256 + D;
  // 16 warps share the register file four to a scheduler (128 each): the producer and the issuers need few, the
  // compute and reduction threads hold 64..128 values at a time. Each role's code follows its own setmaxnreg so that
  // the compiler may use the larger budget there.
  // (setmaxnreg moves registers within what the CTA received at launch, 512 threads x 128: the sum below must fit)
  static_assert(128 * 56 + 384 * 152 <= 512 * 128, "setmaxnreg budget exceeds the launch allocation");
  if (warp < 4) setmaxnreg_dec<56>();

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * Cfg::T_BYTES);
#pragma unroll
      for (int db = 0; db < D / 64; ++db) {
        tma_load_2d(sK + db * AB_SLAB, &tmK, kv_full, hk * D + 64 * db, kv_base + k_first);
        tma_load_2d(sV + db * AB_SLAB, &tmV, kv_full, hk * D + 64 * db, kv_base + k_first);
      }
      bool ok = true;
      int nq_issued = 0, ndo_issued = 0;
      for (int n = 0; n < N && ok; ++n) {
        const int st = n & 1;
        const int r0 = row_base + (i_lo + n) * 128;
        ok = mbar_wait_bounded(&q_empty[st], ((n >> 1) & 1) ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
        if (!ok) break;
        mbar_expect_tx(&q_full[st], Cfg::T_BYTES + 1024);
#pragma unroll
        for (int db = 0; db < D / 64; ++db)
          tma_load_2d(sQ + st * Cfg::T_BYTES + db * AB_SLAB, &tmQ, &q_full[st], hq * D + 64 * db, r0);
        {
          const long long so = ((long long)b * args.Hq + hq) * args.Sq + (long long)(i_lo + n) * 128;
          bulk_load_1d(sStat + st * 1024, args.lse2 + so, 512, &q_full[st]);
          bulk_load_1d(sStat + st * 1024 + 512, args.delta + so, 512, &q_full[st]);
        }
        ++nq_issued;
        ok = mbar_wait_bounded(do_empty, (n & 1) ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
        if (!ok) break;
        mbar_expect_tx(do_full, Cfg::T_BYTES);
#pragma unroll
        for (int db = 0; db < D / 64; ++db)
          tma_load_2d(sDO + db * AB_SLAB, &tmDO, do_full, hq * D + 64 * db, r0);
        ++ndo_issued;
      }
      if (*abort_flag) {
        // let copies in flight land before the CTA retires (bounded)
        const uint64_t t0 = globaltimer_ns();
        bool drained = false;
        while (!drained && globaltimer_ns() - t0 < 20000000ull) {
          drained = mbar_try_wait(kv_full, 0);
          for (int i = 0; i < 2 && drained; ++i) {
            const int c = nq_issued - 1 - i;
            if (c >= 0) drained = drained && mbar_try_wait(&q_full[c & 1], (c >> 1) & 1);
          }
          if (ndo_issued > 0) drained = drained && mbar_try_wait(do_full, (ndo_issued - 1) & 1);
        }
        if (!drained && args.err) atomicCAS(args.err, 0, PT_ERR_TIMEOUT_DRAIN);
      }
    }
  } else if (warp <= 2) {
    // ---------------------------------------------------------------- MMA issuers
    // A thread that issues tcgen05.mma runs nearly in lock step with the tensor core, so the waits, fences and commits
    // of a lone issuer are tensor-core idle time. Two issuers share the work: the "front" (warp 1) issues S^T and dP^T,
    // the "back" (warp 2) dV, dK and dQ. MMAs of one thread execute in order; every hazard between the two threads is
    // covered by a barrier the consumer side already needs (dp_read before the next S^T, dq_read before the next dP^T,
    // p_ready / ds_ready before dV / dK / dQ). Q and dO stages are released when both issuers have committed past them.
    if (lane == 0) {
      constexpr uint32_t IDESC_ST = make_idesc(1, 1, 128, 128, false, false);  // S^T, dP^T: both operands K-major
      constexpr uint32_t IDESC_DV = make_idesc(1, 1, 128, D, false, true);     // A in TMEM, B MN-major
      constexpr uint32_t IDESC_DK = make_idesc(1, 1, 128, D, false, true);     // A K-major smem, B MN-major
      constexpr uint32_t IDESC_DQ = make_idesc(1, 1, 128, D, true, true);      // both MN-major
      // descriptor words of the operand tiles (see smem_desc_lo): "k" = read K-major (rows 128 B apart), "m" = read
      // MN-major (the reduction index walks the rows, 64-element blocks one slab apart)
      constexpr uint32_t HI = smem_desc_hi_sw128(1024);
      const uint32_t k_k = smem_desc_lo(smem_u32(sK), 16), k_m = smem_desc_lo(smem_u32(sK), AB_SLAB);
      const uint32_t v_k = smem_desc_lo(smem_u32(sV), 16);
      const uint32_t do_k = smem_desc_lo(smem_u32(sDO), 16), do_m = smem_desc_lo(smem_u32(sDO), AB_SLAB);
      const uint32_t ds_k = smem_desc_lo(smem_u32(sDS), 16), ds_m = smem_desc_lo(smem_u32(sDS), AB_SLAB);
      const uint32_t q_k0 = smem_desc_lo(smem_u32(sQ), 16), q_m0 = smem_desc_lo(smem_u32(sQ), AB_SLAB);
      bool ok = mbar_wait_bounded(kv_full, 0, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
      if (warp == 1) {
        // ------------------------------------------------ front: S^T(n+1) and dP^T(n)
        auto issue_S = [&](int n) {
          const uint32_t q_k = q_k0 + (n & 1) * (Cfg::T_BYTES >> 4);
          const uint32_t d = tmem_base + (n & 1) * 128;
#pragma unroll
          for (int db = 0; db < D / 64; ++db)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16_lh(d, k_k + ((db * AB_SLAB + k * 32) >> 4), HI, q_k + ((db * AB_SLAB + k * 32) >> 4), HI, IDESC_ST,
                          (db | k) != 0 ? 1u : 0u);
          umma_commit(s_full);
          umma_commit(&q_empty[n & 1]);  // this issuer's share of the release of Q(n)
        };
        if (ok) ok = mbar_wait_bounded(&q_full[0], 0, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
        if (ok) { tc_fence_after(); issue_S(0); }
        for (int n = 0; n < N && ok; ++n) {
          const uint32_t ph = n & 1;
          const uint32_t tRP = tmem_base + (1 - (n & 1)) * 128;
          ok = mbar_wait_bounded(do_full, ph, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          if (n > 0) {
            ok = mbar_wait_bounded(dq_read, (n - 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
            if (!ok) break;
          }
          tc_fence_after();
          // dP^T = V dO^T
#pragma unroll
          for (int db = 0; db < D / 64; ++db)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16_lh(tRP, v_k + ((db * AB_SLAB + k * 32) >> 4), HI, do_k + ((db * AB_SLAB + k * 32) >> 4), HI, IDESC_ST,
                          (db | k) != 0 ? 1u : 0u);
          umma_commit(dp_full);
          umma_commit(do_empty);  // this issuer's share of the release of dO(n)
          // next S^T into the region dP^T has just left
          ok = mbar_wait_bounded(dp_read, ph, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          if (n + 1 < N) {
            ok = mbar_wait_bounded(&q_full[(n + 1) & 1], ((n + 1) >> 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            issue_S(n + 1);
          }
        }
      } else {
        // ------------------------------------------------ back: dV(n), dK(n), dQ(n)
        for (int n = 0; n < N && ok; ++n) {
          const uint32_t ph = n & 1;
          const uint32_t tRS = tmem_base + (n & 1) * 128;
          const uint32_t q_m = q_m0 + (n & 1) * (Cfg::T_BYTES >> 4);
          const uint32_t accn = n != 0 ? 1u : 0u;
          // dV += P^T dO  (P^T packed bf16 in TMEM: query columns 0..63 at +0, 64..127 at +64)
          ok = mbar_wait_bounded(do_full, ph, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          ok = mbar_wait_bounded((n & 1) ? p_ready2 : p_ready, (n >> 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16_ts_lh(tDV, tRS + (k >> 2) * 64 + (k & 3) * 8, do_m + ((k * 2048) >> 4), HI, IDESC_DV, k != 0 ? 1u : accn);
          umma_commit(do_empty);
          // dK += dS^T Q ; dQ = dS K
          ok = mbar_wait_bounded(&q_full[n & 1], (n >> 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          ok = mbar_wait_bounded(ds_ready, ph, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          // dQ first: reading it out and handing its TMEM region to the next dP^T is the longest dependency of a step
          // (dS -> dQ -> read-out -> dP^T -> dS), dK only accumulates
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16_lh(tRS, ds_m + ((k * 2048) >> 4), HI, k_m + ((k * 2048) >> 4), HI, IDESC_DQ, k != 0 ? 1u : 0u);
          umma_commit(dq_full);
#pragma unroll
          for (int g = 0; g < 2; ++g)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16_lh(tDK, ds_k + ((g * AB_SLAB + k * 32) >> 4), HI, q_m + (((g * 4 + k) * 2048) >> 4), HI, IDESC_DK,
                          (g | k) != 0 ? 1u : accn);
          umma_commit(dk_done);
          umma_commit(&q_empty[n & 1]);
        }
        if (ok) umma_commit(all_done);
      }
    }
  } else if (warp == 3) {
    // idle: completes the first warp group
  } else if (warp < 12) {
    // ---------------------------------------------------------------- compute: thread = key row, 64 query columns
    setmaxnreg_inc<152>();
    const int g = (warp - 4) >> 2;            // column half
    const int qd = warp & 3;                  // TMEM lane quarter
    const int r = qd * 32 + lane;             // key row of the tile
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const int kp = k_first + r;               // key position within the batch entry
    const bool key_valid = kp < args.Sk;
    uint8_t* ds_row = sDS + g * AB_SLAB + r * 128;
    for (int n = 0; n < N; ++n) {
      const int i = i_lo + n;
      const int q0 = i * 128 + g * 64;        // first query row of my 64 columns
      const uint32_t ph = n & 1;
      const uint32_t tRS = tmem_base + lane_off + (n & 1) * 128 + g * 64;
      const uint32_t tRP = tmem_base + lane_off + (1 - (n & 1)) * 128 + g * 64;
      // does this (query tile, key tile) pair need element masks?
      bool need_mask = (k_first + 127 >= args.Sk) || (i * 128 + 127 >= args.Sq);
      if (args.causal) need_mask = need_mask || (args.q_off + i * 128 < k_first + 127);
      if (args.row_lo) need_mask = need_mask || (args.row_lo[row_base + min(i * 128 + 127, args.Sq - 1)] > k_first);
      int good = 1;
      if (lane == 0) {
        good = mbar_wait_bounded(s_full, ph, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
        // the row statistics arrived with Q (already complete: S^T has been computed from it)
        if (good) good = mbar_wait_bounded(&q_full[n & 1], (n >> 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) break;
      tc_fence_after();
      const float* st_lse = reinterpret_cast<const float*>(sStat + (n & 1) * 1024) + g * 64;
      const float* st_del = st_lse + 128;
      // Both phases below walk my 64 query columns in two chunks of 32 with the chunk loop kept rolled: fully unrolled,
      // the loop body of a compute warp was ~30 KB of straight-line code, every instruction used once per query tile,
      // and instruction fetch (not a pipe) bounded the warps ("no instruction" was their largest stall reason).
      // P^T chunk c (AB_EXP_CHUNK / 2 packed columns) goes to the columns of my S^T half right after chunk c-1's: the
      // scores there have been read by then.
      // one rolled loop per case: the element masks (diagonal and ragged tiles only) stay out of the common loop
      auto exp_pass = [&](auto masked_c) {
        constexpr bool MASKED = decltype(masked_c)::value;
#pragma unroll 1
        for (int c = 0; c < 64 / AB_EXP_CHUNK; ++c) {
          uint32_t sv[AB_EXP_CHUNK], pk[AB_EXP_CHUNK / 2];
          if (AB_EXP_CHUNK == 32) tmem_ld_32x32(tRS + AB_EXP_CHUNK * c, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
          else tmem_ld_32x16(tRS + AB_EXP_CHUNK * c, *reinterpret_cast<uint32_t(*)[16]>(&sv[0]));
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < AB_EXP_CHUNK / 4; ++u) {
            const float4 ls = *reinterpret_cast<const float4*>(st_lse + c * AB_EXP_CHUNK + u * 4);
            // AB_POLY_MASK chooses, element by element, the polynomial (FMA pipe) or the special-function unit
            const float x0 = fmaf(__uint_as_float(sv[4 * u + 0]), args.scale_log2, -ls.x);
            const float x1 = fmaf(__uint_as_float(sv[4 * u + 1]), args.scale_log2, -ls.y);
            const float x2 = fmaf(__uint_as_float(sv[4 * u + 2]), args.scale_log2, -ls.z);
            const float x3 = fmaf(__uint_as_float(sv[4 * u + 3]), args.scale_log2, -ls.w);
            float p0 = (AB_POLY_MASK & (1u << ((4 * u + 0) & 7))) ? exp2_poly(x0) : ex2_approx(x0);
            float p1 = (AB_POLY_MASK & (1u << ((4 * u + 1) & 7))) ? exp2_poly(x1) : ex2_approx(x1);
            float p2 = (AB_POLY_MASK & (1u << ((4 * u + 2) & 7))) ? exp2_poly(x2) : ex2_approx(x2);
            float p3 = (AB_POLY_MASK & (1u << ((4 * u + 3) & 7))) ? exp2_poly(x3) : ex2_approx(x3);
            if (MASKED) {
              const int qr = q0 + c * AB_EXP_CHUNK + 4 * u;
              const float pv[4] = {p0, p1, p2, p3};
              float po[4];
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                bool vis = key_valid && qr + x < args.Sq;
                if (args.causal) vis = vis && kp <= args.q_off + qr + x;
                if (args.row_lo && vis) vis = kp >= args.row_lo[row_base + qr + x];
                po[x] = vis ? pv[x] : 0.f;
              }
              p0 = po[0]; p1 = po[1]; p2 = po[2]; p3 = po[3];
            }
            pk[2 * u] = pack_bf16x2(p0, p1);
            pk[2 * u + 1] = pack_bf16x2(p2, p3);
          }
          if (AB_EXP_CHUNK == 32) tmem_st_32x16(tRS + (AB_EXP_CHUNK / 2) * c, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
          else tmem_st_32x8(tRS + (AB_EXP_CHUNK / 2) * c, *reinterpret_cast<uint32_t(*)[8]>(&pk[0]));
        }
      };
      if (need_mask) exp_pass(std::true_type{});
      else exp_pass(std::false_type{});
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive((n & 1) ? p_ready2 : p_ready);

      if (lane == 0) {
        good = mbar_wait_bounded(dp_full, ph, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
        // the previous step's dK product (issued after its dQ) must have finished reading the dS^T tile written below
        if (good && n > 0) good = mbar_wait_bounded(dk_done, (n - 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) break;
      tc_fence_after();
      // dS^T = P^T o (dP^T - delta): P^T (as rounded for the dV product) is read back from TMEM, where it stays until
      // the dQ product of this step overwrites the region (issued only after every compute warp has arrived below)
      {
        uint32_t dp[64], pk[32];
        tmem_ld_32x32(tRP, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
        tmem_ld_32x32(tRP + 32, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
        tmem_ld_32x32(tRS, pk);
        tmem_ld_wait();
        // dP^T has left TMEM: the next S^T may be issued into this region
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dp_read);
        // 64 query columns = 8 chunks of 16 bytes in my 128-byte row of the dS^T tile (this part is short: unrolled)
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float4 da = *reinterpret_cast<const float4*>(st_del + t * 8);
          const float4 db = *reinterpret_cast<const float4*>(st_del + t * 8 + 4);
          const float2 pa = unpack_bf16x2(pk[4 * t]), pb = unpack_bf16x2(pk[4 * t + 1]);
          const float2 pc = unpack_bf16x2(pk[4 * t + 2]), pd = unpack_bf16x2(pk[4 * t + 3]);
          uint4 v4;
          v4.x = pack_bf16x2(pa.x * (__uint_as_float(dp[8 * t + 0]) - da.x), pa.y * (__uint_as_float(dp[8 * t + 1]) - da.y));
          v4.y = pack_bf16x2(pb.x * (__uint_as_float(dp[8 * t + 2]) - da.z), pb.y * (__uint_as_float(dp[8 * t + 3]) - da.w));
          v4.z = pack_bf16x2(pc.x * (__uint_as_float(dp[8 * t + 4]) - db.x), pc.y * (__uint_as_float(dp[8 * t + 5]) - db.y));
          v4.w = pack_bf16x2(pd.x * (__uint_as_float(dp[8 * t + 6]) - db.z), pd.y * (__uint_as_float(dp[8 * t + 7]) - db.w));
          *reinterpret_cast<uint4*>(ds_row + ((t ^ (r & 7)) << 4)) = v4;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
  } else {
    // ---------------------------------------------------------------- dQ reduction, then dK / dV
    setmaxnreg_inc<152>();
    const int qd = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    uint8_t* stg = sStg + (warp - 12) * 8192;
    int slot = 0;
    auto stage_out = [&](const uint32_t (&v)[32], const CUtensorMap* tm, int x, int y) {
      uint8_t* st = stg + slot * 4096;
      if (lane == 0) tma_store_wait_read<1>();  // the tile staged two calls ago has been read
      __syncwarp();
      uint8_t* rowp = st + lane * 128;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        uint4 w;
        w.x = v[4 * t]; w.y = v[4 * t + 1]; w.z = v[4 * t + 2]; w.w = v[4 * t + 3];
        *reinterpret_cast<uint4*>(rowp + ((t ^ (lane & 7)) << 4)) = w;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_reduce_add_2d(tm, st, x, y);
        tma_store_commit();
      }
      slot ^= 1;
    };
    bool ok = true;
    for (int n = 0; n < N; ++n) {
      int good = 1;
      if (lane == 0) good = mbar_wait_bounded(dq_full, n & 1, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { ok = false; break; }
      tc_fence_after();
      const uint32_t tR = tmem_base + lane_off + (n & 1) * 128;
      uint32_t v[D / 32][32];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld_32x32(tR + c * 32, v[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_read);
      const int y = row_base + (i_lo + n) * 128 + qd * 32;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) stage_out(v[c], &tmDQ, hq * D + c * 32, y);
    }
    if (ok) {
      int good = 1;
      if (lane == 0) good = mbar_wait_bounded(all_done, 0, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (good) {
        tc_fence_after();
        const int y = kv_base + k_first + qd * 32;
#pragma unroll 1
        for (int c = 0; c < 2 * (D / 32); ++c) {
          const bool is_dv = c >= D / 32;
          const int cc = is_dv ? c - D / 32 : c;
          uint32_t v[32];
          tmem_ld_32x32((is_dv ? tDV : tDK) + lane_off + cc * 32, v);
          tmem_ld_wait();
          stage_out(v, is_dv ? &tmDV : &tmDK, hk * D + cc * 32, y);
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta = rowsum(dO * O), lse2 = lse * log2(e) (+inf where lse is -inf). One thread per 8 elements of a (row, head).
template <int D>
__global__ void attn_bwd_pre_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                    const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2,
                                    int B, int Sq, int Hq, long long ldo, long long lddo) {
  constexpr int TPR = D / 8;  // threads per (row, head)
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long pair = gid / TPR;
  const int part = static_cast<int>(gid % TPR);
  const long long total = (long long)B * Sq * Hq;
  float acc = 0.f;
  long long row = 0;
  int h = 0;
  if (pair < total) {
    row = pair / Hq;
    h = static_cast<int>(pair % Hq);
    const uint4 a = *reinterpret_cast<const uint4*>(out + row * ldo + h * D + part * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(dout + row * lddo + h * D + part * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack_bf16x2(aw[i]), y = unpack_bf16x2(cw[i]);
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
  }
#pragma unroll
  for (int o = TPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (pair < total && part == 0) {
    const long long bb = row / Sq, r = row % Sq;
    const long long idx = (bb * Hq + h) * Sq + r;
    delta[idx] = acc;
    const float l = lse[idx];
    lse2[idx] = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
  }
}

// out[r, c] = bf16(acc[r, c] * scale) over a [rows, cols] fp32 accumulator (8 elements per thread).
__global__ void attn_bwd_post_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, long long n8, float scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4*>(acc)[2 * i], c = reinterpret_cast<const float4*>(acc)[2 * i + 1];
  uint4 w;
  w.x = pack_bf16x2(a.x * scale, a.y * scale);
  w.y = pack_bf16x2(a.z * scale, a.w * scale);
  w.z = pack_bf16x2(c.x * scale, c.y * scale);
  w.w = pack_bf16x2(c.z * scale, c.w * scale);
  reinterpret_cast<uint4*>(out)[i] = w;
}

}  // namespace pt

namespace {
using namespace pt;

template <int D>
int attn_bwd_launch_t(const void* q, const void* k, const void* v, const void* out, const void* dout, const void* lse,
                      void* dq_acc, void* dk_acc, void* dv_acc, float* delta, float* lse2, AttnBwdArgs a, long long ldq,
                      long long ldk, long long ldv, long long ldo, long long lddo, cudaStream_t stream) {
  using Cfg = AttnBwdCfg<D>;
  CUtensorMap tmQ, tmK, tmV, tmDO, tmDQ, tmDK, tmDV;
  const uint64_t rows = (uint64_t)a.B * a.Sq, kv_rows = (uint64_t)a.B * a.Sk;
  if (encode_tmap_2d(&tmQ, q, TM_BF16, rows, (uint64_t)a.Hq * D, ldq, 128, 64, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmK, k, TM_BF16, kv_rows, (uint64_t)a.Hkv * D, ldk, 128, 64, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmV, v, TM_BF16, kv_rows, (uint64_t)a.Hkv * D, ldv, 128, 64, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmDO, dout, TM_BF16, rows, (uint64_t)a.Hq * D, lddo, 128, 64, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmDQ, dq_acc, TM_F32, rows, (uint64_t)a.Hq * D, (uint64_t)a.Hq * D, 32, 32, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmDK, dk_acc, TM_F32, kv_rows, (uint64_t)a.Hkv * D, (uint64_t)a.Hkv * D, 32, 32, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmDV, dv_acc, TM_F32, kv_rows, (uint64_t)a.Hkv * D, (uint64_t)a.Hkv * D, 32, 32, TM_SW_128)) return -3;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return -4;
    configured = true;
  }
  {
    constexpr int TPR = D / 8;
    const long long threads = (long long)a.B * a.Sq * a.Hq * TPR;
    attn_bwd_pre_kernel<D><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout), static_cast<const float*>(lse), delta,
        lse2, a.B, a.Sq, a.Hq, ldo, lddo);
  }
  a.lse2 = lse2;
  a.delta = delta;
  dim3 grid(a.Hq * a.B, (a.Sk + 127) / 128);
  attn_bwd_kernel<D><<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(tmQ, tmK, tmV, tmDO, tmDQ, tmDK, tmDV, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
}  // namespace

// Gradients of pt_attn_fwd. q, k, v, out, dout: bf16 token-major with row pitches (elements); lse [B,Hq,Sq] fp32 from
// the forward. dq_acc [B*Sq, Hq*d], dk_acc, dv_acc [B*Sk, Hkv*d] are fp32 accumulators the caller has zeroed; delta and
// lse2 are fp32 scratch of B*Hq*Sq + 128 elements (the kernel reads whole 128-row tiles). dq / dk / dv receive the
// bf16 results. d in {64, 128} (same for q/k and v).
PT_API int pt_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const void* lse,
                       const void* row_lo, void* dq_acc, void* dk_acc, void* dv_acc, void* dq, void* dk, void* dv, void* delta,
                       void* lse2, int B, int Sq, int Sk, int Hq, int Hkv, int d, long long ldq, long long ldk, long long ldv,
                       long long ldo, long long lddo, float scale, int causal, int q_off, void* stream_) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || Hkv <= 0 || Hq % Hkv != 0 || scale <= 0.f) return -2;
  AttnBwdArgs a;
  a.B = B; a.Sq = Sq; a.Sk = Sk; a.Hq = Hq; a.Hkv = Hkv; a.causal = causal; a.q_off = q_off;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.row_lo = static_cast<const int*>(row_lo);
  a.lse2 = nullptr; a.delta = nullptr;
  a.err = device_status_word();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc;
  if (d == 128)
    rc = attn_bwd_launch_t<128>(q, k, v, out, dout, lse, dq_acc, dk_acc, dv_acc, static_cast<float*>(delta),
                                static_cast<float*>(lse2), a, ldq, ldk, ldv, ldo, lddo, stream);
  else if (d == 64)
    rc = attn_bwd_launch_t<64>(q, k, v, out, dout, lse, dq_acc, dk_acc, dv_acc, static_cast<float*>(delta),
                               static_cast<float*>(lse2), a, ldq, ldk, ldv, ldo, lddo, stream);
  else
    return -2;
  if (rc != 0) return rc;
  const long long nq8 = (long long)B * Sq * Hq * d / 8, nk8 = (long long)B * Sk * Hkv * d / 8;
  attn_bwd_post_kernel<<<(unsigned)((nq8 + 255) / 256), 256, 0, stream>>>(static_cast<const float*>(dq_acc),
                                                                         static_cast<__nv_bfloat16*>(dq), nq8, scale);
  attn_bwd_post_kernel<<<(unsigned)((nk8 + 255) / 256), 256, 0, stream>>>(static_cast<const float*>(dk_acc),
                                                                         static_cast<__nv_bfloat16*>(dk), nk8, scale);
  attn_bwd_post_kernel<<<(unsigned)((nk8 + 255) / 256), 256, 0, stream>>>(static_cast<const float*>(dv_acc),
                                                                         static_cast<__nv_bfloat16*>(dv), nk8, 1.0f);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
