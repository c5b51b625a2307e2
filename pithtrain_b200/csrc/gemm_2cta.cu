// Dense bf16 NT GEMM with 2-CTA tcgen05 tiles (cta_group::2).
//
// Default path of ops/gemm.py: gemm_nt for fresh bf16 outputs (q/k/v/o projections, lm_head, dense MLPs); the
// single-CTA family in gemm.cu serves the accumulating, fp32-output, NN / TN and grouped forms.
//
//   D[M,N] = A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate in TMEM, bf16 out through TMA stores.
//   A pair of CTAs (cluster 2x1x1) owns a 256 x 256 output tile: CTA r loads rows [m0 + 128 r, +128) of A and rows
//   [n0 + 128 r, +128) of B (its half of N) with ordinary, non-multicast TMA loads issued in the .cta_group::2 form,
//   whose completion lands on the leader's (CTA 0) mbarrier. The leader's MMA thread issues
//   tcgen05.mma.cta_group::2 (M = 256, N = 256): the pair's tensor cores read both halves of B from both CTAs' shared
//   memory, so each B byte is loaded from L2 once per pair and each shared-memory byte feeds twice the FLOPs of the
//   single-CTA kernel. Each CTA keeps its 128 accumulator rows in its own TMEM and runs its own epilogue.
//
//   per CTA: warp 0 producer, warp 1 MMA (leader only issues; both allocate TMEM), warps 2..5 epilogue.
//   Barriers live at the same shared-memory offset in both CTAs:
//     full[s]       used in CTA 0: leader producer arrives with expect_tx(both CTAs' bytes)
//     empty[s]      in each CTA: leader MMA commits once to its own copy and once to the peer's (mapa address)
//     tmem_full[b]  in each CTA: same
//     tmem_empty[b] used in CTA 0: the 8 epilogue warps of the pair arrive there (remote arrive from CTA 1)
//
// PTX forms follow the vendored CUTLASS headers (cute/arch/copy_sm100_tma.hpp: SM100_TMA_2SM_LOAD_2D,
// cute/arch/mma_sm100_umma.hpp: SM100_MMA_F16BF16_2x1SM_SS, cute/arch/tmem_allocator_sm100.hpp: Allocator2Sm,
// cutlass/arch/barrier.h: umma_arrive_2x1SM, umma_arrive_2x1SM_sm0).
#include "host_common.h"
#include "ptx.cuh"

namespace pt {

constexpr int T2_BM = 128;  // rows per CTA (256 per pair)
constexpr int T2_BN = 256;  // columns per pair; each CTA loads 128 rows of B
constexpr int T2_BK = 64;
constexpr int T2_STAGES = 5;
constexpr int T2_A_BYTES = T2_BM * T2_BK * 2;        // 16 KB
constexpr int T2_B_BYTES = (T2_BN / 2) * T2_BK * 2;  // 16 KB (this CTA's half)
constexpr int T2_STAGE_BYTES = T2_A_BYTES + T2_B_BYTES;
constexpr int T2_STAGING = 4 * 2 * 4096;
constexpr uint32_t T2_PEER_MASK = 0xFEFFFFFFu;  // clears the pair-rank bit of a shared::cluster address -> CTA 0

struct Gemm2Args {
  int M, N, K;
  int* err;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA load of this CTA's box; completion bytes go to the mbarrier at the same offset in CTA 0.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & T2_PEER_MASK), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrive (once the MMAs issued so far have completed) on the barrier at this offset in both CTAs of the pair: one commit
// per CTA, the peer's copy addressed through mapa (both commits track the same preceding MMAs).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint32_t own = smem_u32(bar);
  uint32_t peer;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(own), "r"(1u));
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(own) : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(peer) : "memory");
}
// Plain arrive on CTA 0's copy of a barrier (from either CTA).
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & T2_PEER_MASK) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmD, const Gemm2Args args) {
  constexpr uint32_t IDESC = make_idesc(1, 1, 2 * T2_BM, T2_BN, false, false);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + T2_STAGES * T2_STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + T2_STAGING);
  uint64_t* empty = full + T2_STAGES;
  uint64_t* tmem_full = empty + T2_STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int m_tiles = (args.M + 2 * T2_BM - 1) / (2 * T2_BM), n_tiles = (args.N + T2_BN - 1) / T2_BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (args.K + T2_BK - 1) / T2_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 8); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc_2cta(tmem_ptr, 512);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  auto tile_origin = [&](int t, int& m0, int& n0) {
    const int GROUP = 8;
    int per = GROUP * n_tiles;
    int gid = t / per, first_m = gid * GROUP;
    int gsz = min(m_tiles - first_m, GROUP);
    int local = t - gid * per;
    m0 = (first_m + local % gsz) * 2 * T2_BM;
    n0 = (local / gsz) * T2_BN;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int m0, n0;
        tile_origin(t, m0, n0);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % T2_STAGES;
          const uint32_t ph = (it / T2_STAGES) & 1;
          ok = mbar_wait_bounded(&empty[s], ph ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_PRODUCER);
          if (!ok) break;
          if (leader) mbar_expect_tx(&full[s], 2 * T2_STAGE_BYTES);
          uint8_t* sa = smem + s * T2_STAGE_BYTES;
          tma_load_2d_pair(sa, &tmA, &full[s], kb * T2_BK, m0 + (int)rank * T2_BM);
          tma_load_2d_pair(sa + T2_A_BYTES, &tmB, &full[s], kb * T2_BK, n0 + (int)rank * (T2_BN / 2));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      uint32_t it = 0, tc = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tc) {
        const int acc = tc & 1;
        ok = mbar_wait_bounded(&tmem_empty[acc], ((tc >> 1) & 1) ^ 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * T2_BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % T2_STAGES;
          ok = mbar_wait_bounded(&full[s], (it / T2_STAGES) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * T2_STAGE_BYTES);
          const uint32_t b_addr = a_addr + T2_A_BYTES;
#pragma unroll
          for (int k = 0; k < T2_BK / 16; ++k)
            umma_f16_pair(d_tmem, make_smem_desc_sw128(a_addr + k * 32, 16, 1024), make_smem_desc_sw128(b_addr + k * 32, 16, 1024),
                          IDESC, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&empty[s]);
        }
        if (!ok) break;
        umma_commit_pair(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    uint32_t tc = 0;
    bool used_tma = false;
    for (int t = pair; t < num_tiles; t += num_pairs, ++tc) {
      int m0, n0;
      tile_origin(t, m0, n0);
      const int acc = tc & 1;
      int good = 1;
      if (lane == 0) good = mbar_wait_bounded(&tmem_full[acc], (tc >> 1) & 1, abort_flag, args.err, PT_ERR_TIMEOUT_EPILOGUE) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * T2_BN;
      const int row0 = m0 + (int)rank * T2_BM + q * 32;
#pragma unroll 1
      for (int cc = 0; cc < T2_BN / 64; ++cc) {
        if (n0 + cc * 64 >= args.N) break;
        uint8_t* st = staging + (q * 2 + (cc & 1)) * 4096;
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(taddr + cc * 64, r0);
        tmem_ld_32x32(taddr + cc * 64 + 32, r1);
        tmem_ld_wait();
        if (cc == T2_BN / 64 - 1 || n0 + (cc + 1) * 64 >= args.N) {
          // the accumulator has left TMEM: hand the buffer back to the leader's MMA thread
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_leader(&tmem_empty[acc]);
        }
        uint8_t* rowp = st + lane * 128;
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
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmD, st, n0 + cc * 64, row0);  // rows or columns past the tensor's extent are clipped by TMA
          tma_store_commit();
          used_tma = true;
        }
      }
    }
    if (lane == 0 && used_tma) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs are done with TMEM and with each other's barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, 512);
  }
}

}  // namespace pt

// x [M, K], w [N, K] bf16 row-major with pitches lda / ldb, out [M, N] bf16 with pitch ldd; K a multiple of 8.
PT_API int pt_gemm2cta_nt(const void* x, const void* w, void* out, int M, int N, int K, long long lda, long long ldb,
                          long long ldd, void* stream_) {
  using namespace pt;
  if (M <= 0 || N <= 0 || K <= 0 || K % 8 != 0) return -2;
  CUtensorMap tmA, tmB, tmD;
  if (encode_tmap_2d(&tmA, x, TM_BF16, M, K, lda, T2_BM, T2_BK, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmB, w, TM_BF16, N, K, ldb, T2_BN / 2, T2_BK, TM_SW_128)) return -3;
  if (encode_tmap_2d(&tmD, out, TM_BF16, M, N, ldd, 32, 64, TM_SW_128)) return -3;
  Gemm2Args a;
  a.M = M; a.N = N; a.K = K;
  a.err = device_status_word();
  const int smem = T2_STAGES * T2_STAGE_BYTES + T2_STAGING + 256 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    configured = true;
  }
  const int m_tiles = (M + 2 * T2_BM - 1) / (2 * T2_BM), n_tiles = (N + T2_BN - 1) / T2_BN;
  int pairs = sm_count() / 2;
  if (pairs > m_tiles * n_tiles) pairs = m_tiles * n_tiles;
  gemm2cta_kernel<<<2 * pairs, 192, smem, static_cast<cudaStream_t>(stream_)>>>(tmA, tmB, tmD, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
