// GQA attention forward for sm_100a, head dim 128, bf16 (tcgen05 / TMEM / TMA): causal self-attention, and the
// unmasked block form that ring attention uses (K/V may then live in another GPU's published buffer).
//
// Status: compiles for sm_100a (63 registers, no spills) but has not been validated on hardware yet, so nothing
// calls it unless PITHTRAIN_OWN_ATTENTION=1 is set (see ops/attention_native.py); the default attention path is the
// library kernel. The role of the reference's FlashAttention-4 forward (pithtrain/operators/flash_attn_v4.py:17-45).
//
//   grid  = (S / 128 query tiles, Hq, B), longest (last) query tile first
//   warp 0      TMA producer : Q tile once, then K and V tiles of 128 keys through two-stage rings
//   warp 1      MMA issuer   : S = Q K^T into one of two TMEM buffers, O += P V into a third
//   warps 2..5  softmax      : one thread per query row (tcgen05.ld 32x32b hands thread t row t of the
//                              warp's lane quarter, so row max / row sum need no shuffles); writes P as
//                              bf16 into a 128B-swizzled K-major shared-memory tile for the PV MMA;
//                              rescales O lazily (only when a row maximum grows by more than 2^8)
//
// Layouts: q [B*S, Hq*128], k/v [B*S, Hkv*128] (token-major, as the qkv projection writes them),
// out [B*S, Hq*128] bf16, lse [B, Hq, S] fp32 (natural log of the scaled scores' sum).
// TMEM: 512 columns = S0 | S1 | O | unused.  Shared memory: Q 32 KB, K 2x32 KB, V 2x32 KB, P 32 KB.
//
// Every wait is bounded (mbar_wait_bounded); on a timeout the roles leave their loops, the CTA frees
// its TMEM and the status word carries the code.
#include "host_common.h"
#include "ptx.cuh"

namespace pt {

constexpr int AT_BM = 128;       // query rows per CTA
constexpr int AT_BN = 128;       // keys per KV tile
constexpr int AT_D = 128;        // head dim
constexpr int AT_KSTAGES = 2;
constexpr int AT_TILE = 128 * 64 * 2;           // one [128 x 64] bf16 swizzle slab: 16 KB
constexpr int AT_Q_BYTES = 2 * AT_TILE;         // D = 128 = two slabs
constexpr int AT_K_BYTES = 2 * AT_TILE;
constexpr int AT_V_BYTES = 2 * AT_TILE;         // two 64-key blocks x (two [64 x 64] boxes)
constexpr int AT_P_BYTES = 2 * AT_TILE;
constexpr float AT_RESCALE_LOG2 = 8.0f;         // tolerated growth of a row maximum before O is rescaled

struct AttnArgs {
  int B, S, Sk, Hq, Hkv;  // S query tokens and Sk key tokens per batch entry
  int causal;            // 1: self-attention with the causal mask (S == Sk); 0: every query sees every key (ring blocks)
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* out;
  long long ldo;     // elements between consecutive tokens of out
  float* lse;
  int* err;
};

__global__ void __launch_bounds__(192, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + AT_Q_BYTES;
  uint8_t* sV = sK + AT_KSTAGES * AT_K_BYTES;
  uint8_t* sP = sV + AT_KSTAGES * AT_V_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + AT_P_BYTES);
  uint64_t* q_full = bars;                  // 1
  uint64_t* k_full = bars + 1;              // 2
  uint64_t* k_empty = bars + 3;             // 2
  uint64_t* v_full = bars + 5;              // 2
  uint64_t* v_empty = bars + 7;             // 2
  uint64_t* s_full = bars + 9;              // 2  MMA -> softmax
  uint64_t* s_empty = bars + 11;            // 2  softmax (4 warps) -> MMA
  uint64_t* p_full = bars + 13;             // 1  softmax (128 threads) -> MMA
  uint64_t* pv_done = bars + 14;            // 1  MMA -> softmax: PV of a tile finished (P free, O readable)
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (args.Hq / args.Hkv);
  const int q0 = qt * AT_BM;
  const int n_kv = args.causal ? qt + 1 : args.Sk / AT_BN;  // causal: key tiles 0..qt
  const int row_base = b * args.S;
  const int kv_base = b * args.Sk;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < AT_KSTAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 4); }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
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
  const uint32_t tS0 = tmem_base, tO = tmem_base + 256;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      mbar_expect_tx(q_full, AT_Q_BYTES);
      tma_load_2d(sQ, &tmQ, q_full, h * AT_D, row_base + q0);
      tma_load_2d(sQ + AT_TILE, &tmQ, q_full, h * AT_D + 64, row_base + q0);
      int issued_k = 0, issued_v = 0;
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % AT_KSTAGES;
        const uint32_t ph = (j / AT_KSTAGES) & 1;
        const int kv0 = kv_base + j * AT_BN;
        ok = mbar_wait_bounded(&k_empty[s], ph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
        if (!ok) break;
        mbar_expect_tx(&k_full[s], AT_K_BYTES);
        tma_load_2d(sK + s * AT_K_BYTES, &tmK, &k_full[s], hk * AT_D, kv0);
        tma_load_2d(sK + s * AT_K_BYTES + AT_TILE, &tmK, &k_full[s], hk * AT_D + 64, kv0);
        ++issued_k;
        ok = mbar_wait_bounded(&v_empty[s], ph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
        if (!ok) break;
        mbar_expect_tx(&v_full[s], AT_V_BYTES);
        // MN-major B operand: per 64-key block, two [64 keys x 64 d] boxes 8 KB apart
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int db = 0; db < 2; ++db)
            tma_load_2d(sV + s * AT_V_BYTES + kb * AT_TILE + db * 8192, &tmV, &v_full[s], hk * AT_D + 64 * db, kv0 + 64 * kb);
        ++issued_v;
      }
      if (*abort_flag) {
        // let copies in flight land before the CTA retires
        uint64_t t0 = globaltimer_ns();
        bool drained = false;
        while (!drained && globaltimer_ns() - t0 < 20000000ull) {
          drained = mbar_try_wait(q_full, 0);
          for (int i = 0; i < AT_KSTAGES && drained; ++i) {
            const int jk = issued_k - 1 - i, jv = issued_v - 1 - i;
            if (jk >= 0) drained = drained && mbar_try_wait(&k_full[jk % AT_KSTAGES], (jk / AT_KSTAGES) & 1);
            if (jv >= 0) drained = drained && mbar_try_wait(&v_full[jv % AT_KSTAGES], (jv / AT_KSTAGES) & 1);
          }
        }
        if (!drained && args.err) atomicCAS(args.err, 0, PT_ERR_TIMEOUT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc(1, 1, AT_BM, AT_BN, false, false);
      constexpr uint32_t IDESC_O = make_idesc(1, 1, AT_BM, AT_D, false, true);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
      auto issue_S = [&](int j) -> bool {
        const int s = j % AT_KSTAGES, sb = j & 1;
        if (!mbar_wait_bounded(&s_empty[sb], ((j >> 1) & 1) ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA)) return false;
        if (!mbar_wait_bounded(&k_full[s], (j / AT_KSTAGES) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * AT_K_BYTES);
#pragma unroll
        for (int db = 0; db < 2; ++db)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tS0 + sb * AT_BN, make_smem_desc_sw128(q_addr + db * AT_TILE + k * 32, 16, 1024),
                     make_smem_desc_sw128(k_addr + db * AT_TILE + k * 32, 16, 1024), IDESC_S, (db | k) != 0 ? 1u : 0u);
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[sb]);
        return true;
      };
      if (ok) ok = issue_S(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) { ok = issue_S(j + 1); if (!ok) break; }
        const int s = j % AT_KSTAGES;
        ok = mbar_wait_bounded(p_full, j & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        ok = mbar_wait_bounded(&v_full[s], (j / AT_KSTAGES) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * AT_V_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tO, make_smem_desc_sw128(p_addr + kb * AT_TILE + k * 32, 16, 1024),
                     make_smem_desc_sw128(v_addr + kb * AT_TILE + k * 2048, 8192, 1024), IDESC_O,
                     (j | kb | k) != 0 ? 1u : 0u);
        umma_commit(&v_empty[s]);
        umma_commit(pv_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax (one thread per row)
    const int q = warp & 3;
    const int r = q * 32 + lane;              // row of the tile
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const int qpos = q0 + r;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int sb = j & 1;
      int good = 1;
      if (lane == 0) good = mbar_wait_bounded(&s_full[sb], (j >> 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { ok = false; break; }
      tc_fence_after();
      const uint32_t tS = tS0 + lane_off + sb * AT_BN;
      const bool diag = args.causal && (j == qt);
      const int kpos0 = j * AT_BN;
      // pass 1: row maximum (log2 domain)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tS + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(v[i]);
          if (diag && kpos0 + c * 32 + i > qpos) x = -INFINITY;
          mx = fmaxf(mx, x);
        }
      }
      const float m_new = fmaxf(m_ref, mx * args.scale_log2);  // scale > 0
      // the previous PV must be done before P is overwritten and before O may be rescaled
      if (j > 0) {
        if (lane == 0) good = mbar_wait_bounded(pv_done, (j - 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { ok = false; break; }
        tc_fence_after();
      }
      const bool grow = m_new > m_ref + AT_RESCALE_LOG2;
      if (j == 0) {
        m_ref = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        // warp-uniform branch: tcgen05.ld/st are warp-collective
        const float alpha = exp2f(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tO + lane_off + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(tO + lane_off + c * 32, v);
        }
        tmem_st_wait();
      }
      // pass 2: p = 2^(s - m_ref), row sum, bf16 P tile (K-major, 128-byte swizzle)
      uint8_t* prow = sP + r * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tS + c * 32, v);
        tmem_ld_wait();
        if (c == 3) {
          // S has left TMEM: hand the buffer back for tile j + 2
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_empty[sb]);
        }
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = fmaf(__uint_as_float(v[i]), args.scale_log2, -m_ref);
          float e = exp2f(x);
          if (diag && kpos0 + c * 32 + i > qpos) e = 0.f;
          p[i] = e;
          l += e;
        }
        uint8_t* blk = prow + (c >> 1) * AT_TILE;  // 64-key block
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint4 w;
          w.x = pack_bf16x2(p[8 * t + 0], p[8 * t + 1]);
          w.y = pack_bf16x2(p[8 * t + 2], p[8 * t + 3]);
          w.z = pack_bf16x2(p[8 * t + 4], p[8 * t + 5]);
          w.w = pack_bf16x2(p[8 * t + 6], p[8 * t + 7]);
          const int chunk = (c & 1) * 4 + t;
          *reinterpret_cast<uint4*>(blk + ((chunk ^ (r & 7)) << 4)) = w;
        }
      }
      tc_fence_before();          // orders the tcgen05.st of a rescale before the MMA thread's PV
      fence_proxy_async_smem();   // generic-proxy writes of P before the async-proxy reads of the MMA
      mbar_arrive(p_full);
    }
    if (ok) {
      int good = 1;
      if (lane == 0) good = mbar_wait_bounded(pv_done, (n_kv - 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (good) {
        tc_fence_after();
        const float inv = 1.f / l;
        __nv_bfloat16* orow = args.out + (long long)(row_base + qpos) * args.ldo + h * AT_D;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tO + lane_off + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[8 * t + 0]) * inv, __uint_as_float(v[8 * t + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(v[8 * t + 2]) * inv, __uint_as_float(v[8 * t + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(v[8 * t + 4]) * inv, __uint_as_float(v[8 * t + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(v[8 * t + 6]) * inv, __uint_as_float(v[8 * t + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + t * 8) = w;
          }
        }
        args.lse[((long long)b * args.Hq + h) * args.S + qpos] = m_ref * 0.6931471805599453f + logf(l);
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
int attn_fwd_launch(const void* q, const void* k, const void* v, void* out, void* lse, int B, int S, int Sk, int Hq, int Hkv,
                    long long ldq, long long ldk, long long ldv, long long ldo, float scale, int causal, void* stream_) {
  using namespace pt;
  if (S <= 0 || Sk <= 0 || S % AT_BM != 0 || Sk % AT_BN != 0 || Hkv <= 0 || Hq % Hkv != 0 || B <= 0 || (causal && S != Sk)) return -2;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t rows = (uint64_t)B * S, kv_rows = (uint64_t)B * Sk;
  if (encode_tmap_2d(&tmQ, q, TM_BF16, rows, (uint64_t)Hq * AT_D, ldq, 128, 64, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmK, k, TM_BF16, kv_rows, (uint64_t)Hkv * AT_D, ldk, 128, 64, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmV, v, TM_BF16, kv_rows, (uint64_t)Hkv * AT_D, ldv, 64, 64, TM_SW_128)) return -3;
  AttnArgs a;
  a.B = B; a.S = S; a.Sk = Sk; a.Hq = Hq; a.Hkv = Hkv; a.causal = causal;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.out = static_cast<__nv_bfloat16*>(out); a.ldo = ldo;
  a.lse = static_cast<float*>(lse);
  a.err = device_status_word();
  const int smem = AT_Q_BYTES + AT_KSTAGES * (AT_K_BYTES + AT_V_BYTES) + AT_P_BYTES + 256 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    configured = true;
  }
  dim3 grid(S / AT_BM, Hq, B);
  attn_fwd_kernel<<<grid, 192, smem, stream>>>(tmQ, tmK, tmV, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
}  // namespace

// q [B*S, Hq*128], k, v [B*S, Hkv*128] bf16 with row pitches ldq / ldk / ldv (elements); S a multiple of 128.
PT_API int pt_attn_fwd_causal(const void* q, const void* k, const void* v, void* out, void* lse, int B, int S, int Hq, int Hkv,
                              long long ldq, long long ldk, long long ldv, long long ldo, float scale, void* stream_) {
  return attn_fwd_launch(q, k, v, out, lse, B, S, S, Hq, Hkv, ldq, ldk, ldv, ldo, scale, 1, stream_);
}

// Block form for ring attention: S query tokens against Sk key tokens per batch entry, no mask. k and v may point
// into another GPU's published buffer (plain, non-multicast TMA loads read it over NVLink), so the block can be
// computed while it is being fetched instead of after a copy.
PT_API int pt_attn_fwd_block(const void* q, const void* k, const void* v, void* out, void* lse, int B, int S, int Sk, int Hq,
                             int Hkv, long long ldq, long long ldk, long long ldv, long long ldo, float scale,
                             void* stream_) {
  return attn_fwd_launch(q, k, v, out, lse, B, S, Sk, Hq, Hkv, ldq, ldk, ldv, ldo, scale, 0, stream_);
}
