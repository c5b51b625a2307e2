// Attention forward for sm_100a (tcgen05 / TMEM / TMA), bf16 in, fp32 accumulate: causal or unmasked, GQA, per-row
// lower key bounds (sliding windows and packed documents), learned per-head sinks, head dims 64, 128, 192/128 (MLA)
// and 256. Takes the role of the reference's FlashAttention-4 forward (pithtrain/operators/flash_attn_v4.py:17-45,
// :58-70). K and V may point into another GPU's published buffer (plain, non-multicast TMA loads), which is how the
// context-parallel ring reads a peer's block while computing on it.
//
//   grid  = (Hq * B, ceil(q tiles / NQ)); a CTA owns NQ (two, where TMEM allows) consecutive 128-row query tiles of one
//           head and walks the key tiles they can see; CTAs with the most key tiles are scheduled first.
//   warp 0          TMA producer : Q tiles once, then K and V tiles of 128 keys through KST-stage rings
//   warps 1..NQ     MMA issuers  : one per query tile: S_t = Q_t K^T into TMEM; O_t += P_t V with P_t read from TMEM
//   warps 4..       softmax, 4 warps per tile, one thread per query row (tcgen05.ld 32x32b hands
//                   thread t row t of the warp's lane quarter, so row max / row sum need no shuffles). The row's 128
//                   scores are held in registers; P is written back over S in TMEM as packed bf16 (64 columns) and
//                   feeds the P V MMA from there, so P never touches shared memory. O is rescaled lazily (only when a
//                   row maximum grows by more than 2^8). The two tiles alternate on the tensor core: while one tile's
//                   softmax runs, the other tile's P V and next S are in flight.
//
// Visibility of key kp for the query at row r (absolute position qpos = q_off + r):
//   lo[r] <= kp <= (causal ? qpos : Sk - 1), with lo[r] = row_lo ? row_lo[b * Sq + r] : 0 (non-decreasing in r).
// Layouts: q [B*Sq, Hq*DQK], k [B*Sk, Hkv*DQK], v [B*Sk, Hkv*DV] (token-major with row pitches), out [B*Sq, Hq*DV]
// bf16, lse [B, Hq, Sq] fp32 (natural log; includes the sink when one is given).
// TMEM: S_0 | S_1 | O_0 | O_1.  Every wait is bounded (mbar_wait_bounded); on a timeout the roles leave their loops,
// the CTA frees its TMEM and the status word carries the code.
#include "host_common.h"
#include "ptx.cuh"

namespace pt {

constexpr int AT_SLAB = 128 * 64 * 2;      // one [128 x 64] bf16 swizzle slab: 16 KB
constexpr float AT_RESCALE_LOG2 = 8.0f;    // tolerated growth of a row maximum before O is rescaled
#ifndef AT_ROLLED
#define AT_ROLLED 0  // 1: softmax passes as rolled loops over 32-key chunks re-read from TMEM (measured 196 us against 189 us)
#endif
#ifndef AT_POLY_MASK
// Which of every 8 scores take the polynomial exp2 on the FMA pipe instead of the special-function unit (bit i =
// element i mod 8). Measured at 1 x 4096 x 32/4 heads x 128, causal: 0x00 210 us, 0x55 216 us, 0xB5 223 us, 0x77 233 us,
// 0xFF 249 us. The polynomial's ~9 issue slots per element cost more than the special-function unit's queueing saves,
// so every exponential stays on that unit; the mask remains as a tuning knob.
#define AT_POLY_MASK 0x00u
#endif

struct AttnArgs {
  int B, Sq, Sk, Hq, Hkv;
  int causal;         // 1: key position <= query position
  int q_off;          // absolute position of query row 0 relative to key 0
  float scale_log2;   // softmax scale * log2(e)
  const int* row_lo;  // optional per-row lower key bound [B*Sq]
  const float* sinks; // optional per-head sink logits [Hq]
  __nv_bfloat16* out;
  long long ldo;      // elements between consecutive tokens of out
  float* lse;
  int* err;
};

template <int DQK, int DV, int NQ, int KST>
struct AttnFwdCfg {
  static constexpr int Q_BYTES = (DQK / 64) * AT_SLAB;
  static constexpr int K_BYTES = Q_BYTES;
  static constexpr int V_BYTES = (DV / 64) * AT_SLAB;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM = NQ * Q_BYTES + KST * (K_BYTES + V_BYTES) + BAR_BYTES + 1024;
  // warp group 0: producer, one MMA warp per tile, idle warps; then one warp group of four softmax warps per tile
  static constexpr int THREADS = 128 + 128 * NQ;
  static_assert(NQ * 128 + NQ * DV <= 512, "TMEM columns");
};


// p = 2^(s * scale - m) for chunks [C0, C1) of the 128 scores of a row (in registers; a chunk = 32 keys), written back
// over the scores' TMEM columns as packed bf16 (chunk c -> columns [16c, 16c+16)); returns their sum. POLY selects which of every 8
// element pairs are evaluated by polynomial on the FMA pipe instead of the special-function unit.
template <uint32_t POLY, int C0, int C1>
__device__ __forceinline__ float softmax_exp_store(const uint32_t (&sv)[128], float scale_log2, float m_use, uint32_t tS) {
  float l4[4] = {0.f, 0.f, 0.f, 0.f};
  const float nm = -m_use;
#pragma unroll
  for (int c = C0; c < C1; ++c) {
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float x0 = fmaf(__uint_as_float(sv[c * 32 + 2 * i]), scale_log2, nm);
      const float x1 = fmaf(__uint_as_float(sv[c * 32 + 2 * i + 1]), scale_log2, nm);
      // POLY bit (2i mod 8) / (2i+1 mod 8): which elements of every 8 go to the FMA pipe
      const float e0 = (POLY & (1u << ((2 * i) & 7))) ? exp2_poly(x0) : ex2_approx(x0);
      const float e1 = (POLY & (1u << ((2 * i + 1) & 7))) ? exp2_poly(x1) : ex2_approx(x1);
      l4[(2 * i) & 3] += e0;
      l4[(2 * i + 1) & 3] += e1;
      w[i] = pack_bf16x2(e0, e1);
    }
    tmem_st_32x16(tS + c * 16, w);
  }
  return (l4[0] + l4[1]) + (l4[2] + l4[3]);
}

template <int DQK, int DV, int NQ, int KST>
__global__ void __launch_bounds__(128 + 128 * NQ, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnArgs args) {
  using Cfg = AttnFwdCfg<DQK, DV, NQ, KST>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + NQ * Cfg::Q_BYTES;
  uint8_t* sV = sK + KST * Cfg::K_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KST * Cfg::V_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // KST (<= 4)
  uint64_t* k_empty = bars + 5;            // KST
  uint64_t* v_full = bars + 9;             // KST
  uint64_t* v_empty = bars + 13;           // KST
  uint64_t* s_full = bars + 17;            // NQ  MMA -> softmax
  uint64_t* p_full = bars + 19;            // NQ  softmax (4 warps) -> MMA: keys 0..63 of P are in TMEM
  uint64_t* o_done = bars + 21;            // NQ  MMA -> softmax: last P V of the tile finished
  uint64_t* turn = bars + 23;              // NQ  issuer -> the other issuer: "my block is issued, yours may follow"
  uint64_t* p_full2 = bars + 25;           // NQ  softmax (4 warps) -> MMA: keys 64..127 of P are in TMEM
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 27);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Blocks start in linear order (x fastest): heads and batch entries run along x and query-tile pairs along y, last
  // pair first, so that under a causal mask the CTAs with the most key tiles start first on every SM and the short
  // ones fill the tail.
  const int pair = gridDim.y - 1 - blockIdx.y;
  const int h = blockIdx.x % args.Hq, b = blockIdx.x / args.Hq;
  const int hk = h / (args.Hq / args.Hkv);
  const int nK = (args.Sk + 127) / 128;
  const int row_base = b * args.Sq;
  const int kv_base = b * args.Sk;

  // key-tile range [lo_t, hi_t) of each query tile; J0..J1 is their union
  int lo_t[NQ], hi_t[NQ];
  int J0 = 1 << 30, J1 = 0;
#pragma unroll
  for (int t = 0; t < NQ; ++t) {
    const int q0 = (pair * NQ + t) * 128;
    lo_t[t] = hi_t[t] = 0;
    if (q0 < args.Sq) {
      const int last = min(q0 + 127, args.Sq - 1);
      int lo = args.row_lo ? args.row_lo[row_base + q0] : 0;
      int hi = args.causal ? min(args.Sk - 1, args.q_off + last) : args.Sk - 1;  // last visible key of the tile
      lo = max(lo, 0);
      if (hi >= lo) { lo_t[t] = lo / 128; hi_t[t] = min(nK, hi / 128 + 1); }
      if (hi_t[t] > lo_t[t]) { J0 = min(J0, lo_t[t]); J1 = max(J1, hi_t[t]); }
    }
  }
  if (J1 == 0) J0 = 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KST; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], NQ);   // every MMA warp releases a stage
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], NQ);
    }
    for (int t = 0; t < NQ; ++t) {
      mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 4); mbar_init(&p_full2[t], 4); mbar_init(&o_done[t], 1);
      mbar_init(&turn[t], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  if (NQ == 2) {
    // 12 warps share the register file three to a scheduler (168 each). The softmax threads hold a whole score row and
    // need independent exponentials in flight; the producer, the issuers and the idle warp need few registers.
    // Each role's code follows its own setmaxnreg so that the compiler may use the larger budget there.
    // setmaxnreg moves registers within what the CTA received at launch (384 threads x 168 as compiled): a request
    // beyond that pool would wait for ever
    static_assert(NQ != 2 || 128 * 72 + 256 * 216 <= 384 * 168, "setmaxnreg budget exceeds the launch allocation");
    if (warp < 4) setmaxnreg_dec<72>();
  }

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0 && J1 > J0) {
      int nq_act = 0;
#pragma unroll
      for (int t = 0; t < NQ; ++t) nq_act += (hi_t[t] > lo_t[t]) ? 1 : 0;
      mbar_expect_tx(q_full, nq_act * Cfg::Q_BYTES);
#pragma unroll
      for (int t = 0; t < NQ; ++t)
        if (hi_t[t] > lo_t[t])
#pragma unroll
          for (int db = 0; db < DQK / 64; ++db)
            tma_load_2d(sQ + t * Cfg::Q_BYTES + db * AT_SLAB, &tmQ, q_full, h * DQK + 64 * db, row_base + (pair * NQ + t) * 128);
      int issued = 0;
      bool ok = true;
      for (int j = J0; j < J1 && ok; ++j, ++issued) {
        const int s = issued % KST;
        const uint32_t ph = (issued / KST) & 1;
        const int kv0 = kv_base + j * 128;
        ok = mbar_wait_bounded(&k_empty[s], ph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
        if (!ok) break;
        mbar_expect_tx(&k_full[s], Cfg::K_BYTES);
#pragma unroll
        for (int db = 0; db < DQK / 64; ++db)
          tma_load_2d(sK + s * Cfg::K_BYTES + db * AT_SLAB, &tmK, &k_full[s], hk * DQK + 64 * db, kv0);
        ok = mbar_wait_bounded(&v_empty[s], ph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
        if (!ok) break;
        mbar_expect_tx(&v_full[s], Cfg::V_BYTES);
#pragma unroll
        for (int db = 0; db < DV / 64; ++db)
          tma_load_2d(sV + s * Cfg::V_BYTES + db * AT_SLAB, &tmV, &v_full[s], hk * DV + 64 * db, kv0);
      }
      if (*abort_flag) {
        // let copies in flight land before the CTA retires (bounded)
        const uint64_t t0 = globaltimer_ns();
        bool drained = false;
        while (!drained && globaltimer_ns() - t0 < 20000000ull) {
          drained = mbar_try_wait(q_full, 0);
          for (int i = 0; i < KST && drained; ++i) {
            const int c = issued - 1 - i;
            if (c >= 0) {
              drained = drained && mbar_try_wait(&k_full[c % KST], (c / KST) & 1);
              drained = drained && mbar_try_wait(&v_full[c % KST], (c / KST) & 1);
            }
          }
        }
        if (!drained && args.err) atomicCAS(args.err, 0, PT_ERR_TIMEOUT_DRAIN);
      }
    }
  } else if (warp <= NQ) {
    // ---------------------------------------------------------------- MMA issuers, one warp (one thread) per query tile
    // A thread that issues tcgen05.mma runs nearly in lock step with the tensor core (the queue behind it is short), so
    // every barrier wait, fence and commit of a lone issuer is tensor-core idle time. With one issuer per tile the MMAs
    // of one tile run while the other issuer does its bookkeeping. The K / V stages are released when both issuers
    // have committed past them.
    // The issuers take turns, block by block (a block = P V of step j and S of step j+1 of one tile): tile 0, tile 1,
    // tile 0, ... Left alone, both tiles fall into the same phase (their softmax warps share the special-function
    // unit, finish together and hand both blocks to the tensor core at once), and then the tensor core idles through
    // every softmax and the softmax warps through every block: measured 5700 cycles per step of the pair, where the
    // MMAs take 2048. With the turns the softmax of one tile runs under the other tile's block.
    const int t = warp - 1;
    if (lane == 0 && J1 > J0) {
      constexpr uint32_t IDESC_S = make_idesc(1, 1, 128, 128, false, false);
      constexpr uint32_t IDESC_O = make_idesc(1, 1, 128, DV, false, true);
      const int lo = lo_t[t], hi = hi_t[t];
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
      // descriptor words of the operand tiles: a stage or a k-step moves only the low word
      constexpr uint32_t HI = smem_desc_hi_sw128(1024);
      const uint32_t a_lo = smem_desc_lo(smem_u32(sQ + t * Cfg::Q_BYTES), 16), k_lo0 = smem_desc_lo(smem_u32(sK), 16);
      const uint32_t v_lo0 = smem_desc_lo(smem_u32(sV), AT_SLAB);
      const uint32_t tS = tmem_base + t * 128, tO = tmem_base + NQ * 128 + t * DV;
      // A stage is released through tcgen05.commit (arrives once this thread's MMAs so far have completed); an issuer
      // whose tile does not exist (odd tile count) has no MMA to wait for and arrives directly.
      const bool any = hi > lo;
      auto release = [&](uint64_t* bar) { if (any) umma_commit(bar); else mbar_arrive(bar); };
      // S_t(j) = Q_t K_j^T when the tile sees key tile j; the K stage is released either way
      auto step_S = [&](int j) -> bool {
        const int c = j - J0, s = c % KST;
        // every issuer follows the ring stage by stage, also past tiles it does not use: a stage's release counts one
        // arrival per issuer, so nobody may run a full ring ahead
        if (!mbar_wait_bounded(&k_full[s], (c / KST) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA)) return false;
        if (j >= lo && j < hi) {
          tc_fence_after();
          const uint32_t b_lo = k_lo0 + s * (Cfg::K_BYTES >> 4);
#pragma unroll
          for (int db = 0; db < DQK / 64; ++db)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16_lh(tS, a_lo + ((db * AT_SLAB + k * 32) >> 4), HI, b_lo + ((db * AT_SLAB + k * 32) >> 4), HI, IDESC_S,
                          (db | k) != 0 ? 1u : 0u);
          umma_commit(&s_full[t]);
        }
        release(&k_empty[s]);
        return true;
      };
      if (ok) ok = step_S(J0);
      for (int j = J0; j < J1 && ok; ++j) {
        const int c = j - J0, s = c % KST;
        if (NQ == 2) {
          // tile 0 opens step c once tile 1 has issued its block of step c-1; tile 1 follows tile 0 within the step
          if (t == 1) ok = mbar_wait_bounded(&turn[1], c & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          else if (c > 0) ok = mbar_wait_bounded(&turn[0], (c - 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
        }
        ok = mbar_wait_bounded(&v_full[s], (c / KST) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        if (j >= lo && j < hi) {
          ok = mbar_wait_bounded(&p_full[t], (j - lo) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          const uint32_t b_lo = v_lo0 + s * (Cfg::V_BYTES >> 4);
          const uint32_t acc0 = (j != lo) ? 1u : 0u;
          // the softmax warps hand P over in two halves of 64 keys: the first half's MMAs run under the second's exponentials
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ts_lh(tO, tS + k * 8, b_lo + ((k * 2048) >> 4), HI, IDESC_O, k != 0 ? 1u : acc0);
          ok = mbar_wait_bounded(&p_full2[t], (j - lo) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 4; k < 8; ++k)
            umma_f16_ts_lh(tO, tS + k * 8, b_lo + ((k * 2048) >> 4), HI, IDESC_O, 1u);
          if (j == hi - 1) umma_commit(&o_done[t]);
        }
        release(&v_empty[s]);
        if (j + 1 < J1) ok = step_S(j + 1);
        if (NQ == 2) mbar_arrive(&turn[1 - t]);
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax (one thread per row)
    if (NQ == 2) setmaxnreg_inc<216>();
    const int t = (warp - 4) >> 2;            // query tile of this warp group
    const int q = warp & 3;                   // TMEM lane quarter this warp may access
    const int r = q * 32 + lane;              // row of the tile
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const int qrow = (pair * NQ + t) * 128 + r;        // row within the batch entry
    const bool row_valid = qrow < args.Sq;
    const int jlo = lo_t[t], jhi = hi_t[t];
    int lo_row = 0, hi_row = -1;
    if (row_valid) {
      lo_row = args.row_lo ? max(args.row_lo[row_base + qrow], 0) : 0;
      hi_row = args.causal ? min(args.Sk - 1, args.q_off + qrow) : args.Sk - 1;
    }
    const uint32_t tS = tmem_base + lane_off + t * 128;
    const uint32_t tO = tmem_base + lane_off + NQ * 128 + t * DV;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = jlo; j < jhi; ++j) {
      int good = 1;
      if (lane == 0) good = mbar_wait_bounded(&s_full[t], (j - jlo) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { ok = false; break; }
      tc_fence_after();
#if AT_ROLLED
      // Both passes over the 128 scores of the row (maximum, then exponentials) walk four chunks of 32 keys with the
      // chunk loop kept rolled and read each chunk from TMEM when they need it: the straight-line form of this loop
      // body is several times larger, and every instruction of it is fetched once per key tile.
      const int kpos0 = j * 128;
      const bool masked = kpos0 < lo_row || kpos0 + 127 > hi_row;
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32(tS + c * 32, sv);
        tmem_ld_wait();
        if (masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kpos0 + 32 * c + i < lo_row || kpos0 + 32 * c + i > hi_row) sv[i] = 0xff800000u;  // -inf
        }
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx4[u] = fmaxf(mx4[u], fmaxf(__uint_as_float(sv[i + 2 * u]), __uint_as_float(sv[i + 2 * u + 1])));
        }
      }
#else
      // The scores arrive in four chunks of 32 keys; the row maximum of a chunk is taken while the next chunk loads
      // (four independent chains: a thread has little other work to hide a 128-long dependency).
      uint32_t sv[128];
      const int kpos0 = j * 128;
      const bool masked = kpos0 < lo_row || kpos0 + 127 > hi_row;
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      tmem_ld_32x32(tS, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld_wait();
        if (c + 1 < 4) tmem_ld_32x32(tS + (c + 1) * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32 * (c + 1)]));
        if (masked) {
#pragma unroll
          for (int i = 32 * c; i < 32 * c + 32; ++i)
            if (kpos0 + i < lo_row || kpos0 + i > hi_row) sv[i] = 0xff800000u;  // -inf
        }
#pragma unroll
        for (int i = 32 * c; i < 32 * c + 32; i += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx4[u] = fmaxf(mx4[u], fmaxf(__uint_as_float(sv[i + 2 * u]), __uint_as_float(sv[i + 2 * u + 1])));
        }
      }
#endif
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_ref, mx * args.scale_log2);  // scale > 0
      // The S MMA of this step was issued after the P V MMA of the previous one, so O is stable here.
      const bool grow = m_new > m_ref + AT_RESCALE_LOG2;
      if (j == jlo) {
        m_ref = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        // warp-uniform branch: tcgen05.ld/st are warp-collective
        const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
#pragma unroll 1
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tO + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(tO + c * 32, v);
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // masked tiles need exact zeros, which only the special-function path gives; the others put a share of the
      // exponentials on the FMA pipe
      // (the choice is made per warp: the TMEM stores inside are warp-collective)
#if AT_ROLLED
      {
        const float nm = -m_use;
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t sv[32], w[16];
          tmem_ld_32x32(tS + c * 32, sv);
          tmem_ld_wait();
          if (masked) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kpos0 + 32 * c + i < lo_row || kpos0 + 32 * c + i > hi_row) sv[i] = 0xff800000u;  // -inf
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float e0 = ex2_approx(fmaf(__uint_as_float(sv[2 * i]), args.scale_log2, nm));
            const float e1 = ex2_approx(fmaf(__uint_as_float(sv[2 * i + 1]), args.scale_log2, nm));
            l4[(2 * i) & 3] += e0;
            l4[(2 * i + 1) & 3] += e1;
            w[i] = pack_bf16x2(e0, e1);
          }
          // P chunk c -> columns [16c, 16c+16): the scores that were there belong to chunks already read
          tmem_st_32x16(tS + c * 16, w);
          if (c == 1) {
            // first 64 keys of P are complete: their P V MMAs may start under the other half's exponentials
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[t]);
          }
        }
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
      }
#else
      const bool any_masked = __any_sync(0xffffffffu, masked);
      if (any_masked) l += softmax_exp_store<0u, 0, 2>(sv, args.scale_log2, m_use, tS);
      else l += softmax_exp_store<AT_POLY_MASK, 0, 2>(sv, args.scale_log2, m_use, tS);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      if (any_masked) l += softmax_exp_store<0u, 2, 4>(sv, args.scale_log2, m_use, tS);
      else l += softmax_exp_store<AT_POLY_MASK, 2, 4>(sv, args.scale_log2, m_use, tS);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
#endif
      if (lane == 0) mbar_arrive(&p_full2[t]);
    }
    if (ok) {
      int good = 1;
      if (jhi > jlo) {
        if (lane == 0) good = mbar_wait_bounded(&o_done[t], 0, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
      }
      if (good && (pair * NQ + t) * 128 < args.Sq) {
        tc_fence_after();
        float lt = l, mr = m_ref;
        if (args.sinks) {
          const float s2 = args.sinks[h] * 1.4426950408889634f;
          if (mr == -INFINITY) { mr = s2; lt = 1.f; }
          else lt += exp2f(s2 - mr);
        }
        const float inv = lt > 0.f ? 1.f / lt : 0.f;
        __nv_bfloat16* orow = args.out + (long long)(row_base + qrow) * args.ldo + h * DV;
#pragma unroll 1
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t v[32];
          if (jhi > jlo) {
            tmem_ld_32x32(tO + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (row_valid) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(v[8 * u + 0]) * inv, __uint_as_float(v[8 * u + 1]) * inv);
              w.y = pack_bf16x2(__uint_as_float(v[8 * u + 2]) * inv, __uint_as_float(v[8 * u + 3]) * inv);
              w.z = pack_bf16x2(__uint_as_float(v[8 * u + 4]) * inv, __uint_as_float(v[8 * u + 5]) * inv);
              w.w = pack_bf16x2(__uint_as_float(v[8 * u + 6]) * inv, __uint_as_float(v[8 * u + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = w;
            }
          }
        }
        if (row_valid)
          args.lse[((long long)b * args.Hq + h) * args.Sq + qrow] = lt > 0.f ? mr * 0.6931471805599453f + logf(lt) : -INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace pt

namespace {
using namespace pt;

template <int DQK, int DV, int NQ, int KST>
int attn_fwd_launch_t(const void* q, const void* k, const void* v, const AttnArgs& a, long long ldq, long long ldk,
                      long long ldv, cudaStream_t stream) {
  using Cfg = AttnFwdCfg<DQK, DV, NQ, KST>;
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t rows = (uint64_t)a.B * a.Sq, kv_rows = (uint64_t)a.B * a.Sk;
  if (encode_tmap_2d(&tmQ, q, TM_BF16, rows, (uint64_t)a.Hq * DQK, ldq, 128, 64, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmK, k, TM_BF16, kv_rows, (uint64_t)a.Hkv * DQK, ldk, 128, 64, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmV, v, TM_BF16, kv_rows, (uint64_t)a.Hkv * DV, ldv, 128, 64, TM_SW_128)) return -3;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<DQK, DV, NQ, KST>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) !=
        cudaSuccess)
      return -4;
    configured = true;
  }
  const int nQ = (a.Sq + 127) / 128;
  dim3 grid(a.Hq * a.B, (nQ + NQ - 1) / NQ);
  attn_fwd_kernel<DQK, DV, NQ, KST><<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(tmQ, tmK, tmV, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
}  // namespace

// q [B*Sq, Hq*dqk], k [B*Sk, Hkv*dqk], v [B*Sk, Hkv*dv] bf16 with row pitches ldq / ldk / ldv (elements, multiples of
// 8, 16-byte aligned bases). (dqk, dv) in {(64,64), (128,128), (192,128), (256,256)}. row_lo (int32 [B*Sq]) and sinks
// (fp32 [Hq]) may be null. Returns 0, or a negative code for unsupported arguments / launch failures.
PT_API int pt_attn_fwd(const void* q, const void* k, const void* v, void* out, void* lse, const void* row_lo, const void* sinks,
                       int B, int Sq, int Sk, int Hq, int Hkv, int dqk, int dv, long long ldq, long long ldk, long long ldv,
                       long long ldo, float scale, int causal, int q_off, void* stream_) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || Hkv <= 0 || Hq % Hkv != 0 || scale <= 0.f) return -2;
  AttnArgs a;
  a.B = B; a.Sq = Sq; a.Sk = Sk; a.Hq = Hq; a.Hkv = Hkv; a.causal = causal; a.q_off = q_off;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.row_lo = static_cast<const int*>(row_lo);
  a.sinks = static_cast<const float*>(sinks);
  a.out = static_cast<__nv_bfloat16*>(out); a.ldo = ldo;
  a.lse = static_cast<float*>(lse);
  a.err = device_status_word();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (dqk == 128 && dv == 128) return attn_fwd_launch_t<128, 128, 2, 2>(q, k, v, a, ldq, ldk, ldv, stream);
  if (dqk == 64 && dv == 64) return attn_fwd_launch_t<64, 64, 2, 3>(q, k, v, a, ldq, ldk, ldv, stream);
  if (dqk == 192 && dv == 128) return attn_fwd_launch_t<192, 128, 1, 2>(q, k, v, a, ldq, ldk, ldv, stream);
  if (dqk == 256 && dv == 256) return attn_fwd_launch_t<256, 256, 1, 1>(q, k, v, a, ldq, ldk, ldv, stream);
  return -2;
}
