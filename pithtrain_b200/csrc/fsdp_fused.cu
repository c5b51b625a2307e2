// Shard-group collectives over peer memory: reduce-scatter of the flat gradient buffer fused with
// averaging and the gradient-norm partial sums, and the publication of updated parameter regions
// (the all-gather) as direct stores into every peer's flat parameter buffer.
//
// Every rank of a shard group keeps the whole flat gradient / parameter buffer in symmetric
// (CUDA-IPC mapped) memory. The owner of region r
//   1. waits until every peer has flagged "my gradients are final" (flags are system-scope
//      release/acquire words in a small symmetric control block; every wait is bounded),
//   2. reads region r of every peer's gradient buffer with plain loads over NVLink, sums in fp32 in
//      rank order (deterministic), scales by 1/W, writes the result into its own region and
//      accumulates sum(g^2) for the global gradient norm in the same pass,
//   3. flags "done reading" back, which is what a peer waits for before it zeroes its buffer.
// After the optimizer updated the owned region, `push` stores it into the same offsets of every
// peer's parameter buffer and flags "region published"; the next forward waits for W flags.
//
// Takes the role of FSDP2's reduce-scatter / all-gather in the reference (configured at
// pithtrain/modules/training.py:328-376, triggered at pithtrain/dualpipe/dualpipev.py:645-649) and of
// the separate grad-norm pass (pithtrain/tasks/pretrain_lm.py:125-153).
#include <cuda_bf16.h>

#include "host_common.h"
#include "ptx.cuh"
#include "peer_wait.cuh"

namespace pt {
namespace fsdp {

constexpr int MAXW = 32;
// control block layout (unsigned words)
constexpr int CTL_READY = 0, CTL_ACK = 32, CTL_PUSHED = 64, CTL_TICKET = 96, CTL_WORDS = 128;

struct Chan {
  int W, rank, fp32;       // group size, this rank, gradient dtype (1 = fp32, 0 = bf16)
  long long region;        // elements per region
  void* grad[MAXW];        // flat gradient buffer of every rank (own entry = local pointer)
  void* param[MAXW];       // flat parameter buffer (bf16 or fp32, `param_bytes` per element)
  unsigned* ctl[MAXW];     // control block of every rank
  int param_bytes;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ bool wait_ge_bounded(const unsigned* p, unsigned want, int* err) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
    if ((it & 255u) == 255u) {
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > pt_peer_wait_limit_ns) {
        if (err) atomicCAS(err, 0, PT_ERR_TIMEOUT_PEER);
        return false;
      }
    }
    __nanosleep(64);
  }
}

// word[slot + rank] = epoch in every peer's control block (after all prior work of this stream).
__global__ void signal_kernel(Chan c, int slot, unsigned epoch) {
  __threadfence_system();
  if ((int)threadIdx.x < c.W) st_release_sys(c.ctl[threadIdx.x] + slot + c.rank, epoch);
}

// Wait until all W words of `slot` in the local control block reached `epoch`.
__global__ void wait_kernel(Chan c, int slot, unsigned epoch, int* err) {
  if ((int)threadIdx.x < c.W) wait_ge_bounded(c.ctl[c.rank] + slot + threadIdx.x, epoch, err);
}

__global__ void __launch_bounds__(256)
reduce_kernel(Chan c, unsigned epoch, float scale, double* sumsq_partials, int* err) {
  __shared__ int ok_s;
  __shared__ double red[8];
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < c.W) {
    if (!wait_ge_bounded(c.ctl[c.rank] + CTL_READY + threadIdx.x, epoch, err)) ok_s = 0;
  }
  __syncthreads();
  const bool ok = ok_s != 0;
  double local = 0.0;
  if (ok) {
    const int per = c.fp32 ? 4 : 8;  // elements per 16-byte vector
    const long long nvec = c.region / per;
    const long long base_bytes = (long long)c.rank * c.region * (c.fp32 ? 4 : 2);
    // Four vectors per thread and iteration: all W x 4 loads are issued before the first add, so a thread
    // keeps 4 W independent 16-byte loads in flight (peer loads take microseconds over NVLink).
    constexpr int U = 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += U * stride) {
      uint4 raw[U][MAXW > 8 ? 8 : MAXW];
      float acc[U][8];
      const int Wc = c.W;
      for (int rb = 0; rb < Wc; rb += 8) {  // groups of up to 8 ranks keep the register footprint bounded
        const int rn = min(8, Wc - rb);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + u * stride;
          if (v < nvec) {
            for (int r = 0; r < rn; ++r) {
              const char* src = reinterpret_cast<const char*>(c.grad[rb + r]) + base_bytes + v * 16;
              raw[u][r] = (rb + r == c.rank) ? *reinterpret_cast<const uint4*>(src) : ld_cg_v4(src);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (rb == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
          }
          const long long v = v0 + u * stride;
          if (v < nvec) {
            for (int r = 0; r < rn; ++r) {
              const uint4 x = raw[u][r];
              if (c.fp32) {
                acc[u][0] += __uint_as_float(x.x); acc[u][1] += __uint_as_float(x.y);
                acc[u][2] += __uint_as_float(x.z); acc[u][3] += __uint_as_float(x.w);
              } else {
                float2 a = unpack_bf16x2(x.x), b = unpack_bf16x2(x.y), d = unpack_bf16x2(x.z), e = unpack_bf16x2(x.w);
                acc[u][0] += a.x; acc[u][1] += a.y; acc[u][2] += b.x; acc[u][3] += b.y;
                acc[u][4] += d.x; acc[u][5] += d.y; acc[u][6] += e.x; acc[u][7] += e.y;
              }
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * stride;
        if (v >= nvec) continue;
        char* dst = reinterpret_cast<char*>(c.grad[c.rank]) + base_bytes + v * 16;
        uint4 o;
        if (c.fp32) {
          float f0 = acc[u][0] * scale, f1 = acc[u][1] * scale, f2 = acc[u][2] * scale, f3 = acc[u][3] * scale;
          o = make_uint4(__float_as_uint(f0), __float_as_uint(f1), __float_as_uint(f2), __float_as_uint(f3));
          local += (double)f0 * f0 + (double)f1 * f1 + (double)f2 * f2 + (double)f3 * f3;
        } else {
          o.x = pack_bf16x2(acc[u][0] * scale, acc[u][1] * scale); o.y = pack_bf16x2(acc[u][2] * scale, acc[u][3] * scale);
          o.z = pack_bf16x2(acc[u][4] * scale, acc[u][5] * scale); o.w = pack_bf16x2(acc[u][6] * scale, acc[u][7] * scale);
          // the norm is taken of the values as stored (rounded to bf16), like a separate pass would see
          float2 a = unpack_bf16x2(o.x), b = unpack_bf16x2(o.y), d = unpack_bf16x2(o.z), e = unpack_bf16x2(o.w);
          local += (double)a.x * a.x + (double)a.y * a.y + (double)b.x * b.x + (double)b.y * b.y +
                   (double)d.x * d.x + (double)d.y * d.y + (double)e.x * e.x + (double)e.y * e.y;
        }
        *reinterpret_cast<uint4*>(dst) = o;
      }
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < 8; ++i) t += red[i];
    sumsq_partials[blockIdx.x] = t;
    __threadfence();
    unsigned* ticket = c.ctl[c.rank] + CTL_TICKET;
    unsigned n = atomicAdd(ticket, 1u);
    if (n == gridDim.x - 1) {
      *ticket = 0;
      __threadfence_system();
      // every block of this rank finished reading the peers' buffers
      for (int r = 0; r < c.W; ++r) st_release_sys(c.ctl[r] + CTL_ACK + c.rank, epoch);
    }
  }
}

__global__ void __launch_bounds__(256)
push_kernel(Chan c, unsigned epoch) {
  const long long bytes = c.region * c.param_bytes;
  const long long nvec = bytes / 16;
  const long long base = (long long)c.rank * bytes;
  const char* src = reinterpret_cast<const char*>(c.param[c.rank]) + base;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    uint4 u = *reinterpret_cast<const uint4*>(src + v * 16);
    for (int r = 0; r < c.W; ++r) {
      if (r == c.rank) continue;
      *reinterpret_cast<uint4*>(reinterpret_cast<char*>(c.param[r]) + base + v * 16) = u;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned* ticket = c.ctl[c.rank] + CTL_TICKET + 1;
    unsigned n = atomicAdd(ticket, 1u);
    if (n == gridDim.x - 1) {
      *ticket = 0;
      __threadfence_system();
      for (int r = 0; r < c.W; ++r) st_release_sys(c.ctl[r] + CTL_PUSHED + c.rank, epoch);
    }
  }
}

}  // namespace fsdp
}  // namespace pt

PT_API int pt_fsdp_chan_struct_size() { return (int)sizeof(pt::fsdp::Chan); }
PT_API int pt_fsdp_ctl_bytes() { return pt::fsdp::CTL_WORDS * 4; }
PT_API int pt_fsdp_reduce_grid() { return pt::sm_count() * 2; }

// "My gradients are final": flag every peer (stream-ordered after the backward pass).
PT_API int pt_fsdp_signal_ready(const void* chan, unsigned epoch, void* stream) {
  using namespace pt::fsdp;
  signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*reinterpret_cast<const Chan*>(chan), CTL_READY, epoch);
  return (int)cudaGetLastError();
}

// Reduce this rank's region over all peers: grad_local[region] = scale * sum_r grad_r[region];
// sumsq_partials [pt_fsdp_reduce_grid()] doubles receive sum(g^2) of the result.
PT_API int pt_fsdp_reduce_scatter(const void* chan, unsigned epoch, float scale, double* sumsq_partials, void* stream) {
  using namespace pt::fsdp;
  const Chan& c = *reinterpret_cast<const Chan*>(chan);
  if (c.region % 8 != 0) return -2;
  reduce_kernel<<<pt::sm_count() * 2, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(c, epoch, scale, sumsq_partials,
                                                                                       pt::device_status_word());
  return (int)cudaGetLastError();
}

// Before this rank overwrites its gradient buffer: every owner must have finished reading it.
PT_API int pt_fsdp_wait_acks(const void* chan, unsigned epoch, void* stream) {
  using namespace pt::fsdp;
  wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*reinterpret_cast<const Chan*>(chan), CTL_ACK, epoch,
                                                                   pt::device_status_word());
  return (int)cudaGetLastError();
}

// Store the owned parameter region into every peer's buffer, then flag it published.
PT_API int pt_fsdp_push_params(const void* chan, unsigned epoch, void* stream) {
  using namespace pt::fsdp;
  const Chan& c = *reinterpret_cast<const Chan*>(chan);
  if ((c.region * c.param_bytes) % 16 != 0) return -2;
  push_kernel<<<pt::sm_count() * 2, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(c, epoch);
  return (int)cudaGetLastError();
}

// Before the next forward: all W regions of the local parameter buffer are published.
PT_API int pt_fsdp_wait_params(const void* chan, unsigned epoch, void* stream) {
  using namespace pt::fsdp;
  wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*reinterpret_cast<const Chan*>(chan), CTL_PUSHED, epoch,
                                                                   pt::device_status_word());
  return (int)cudaGetLastError();
}

// Sets this translation unit's copy of the peer-wait limit on the current device (see peer_wait.cuh).
extern "C" int pt_fsdp_set_wait_limit(unsigned long long ns) { return pt::set_peer_wait_limit_here(ns); }
