// Expert-parallel exchange over NVLink peer memory: no NCCL, no host synchronisation.
//
// Every rank owns a symmetric "channel" buffer that all peers have mapped. Its data area is
// partitioned by source rank (capacity `cap` rows each), so a sender never needs to know what
// other senders do: it gathers its de-duplicated rows by index and stores them straight into the
// destination's partition (P2P st over NVLink), then publishes a row count and an epoch flag with
// release semantics. The receiver waits (bounded) on the flags, compacts the partitions into one
// dense tensor with a device-side count, and acknowledges so the slot can be reused two epochs
// later (two slots per channel). The return direction (combine, and the gradient of dispatch)
// writes each row back into the (rank, position) cell it came from; the home rank sums a token's
// cells with the ordinary gather-reduce kernel.
//
// Replaces the reference's metadata all-to-all + host read-back + NCCL all_to_all_single
// (pithtrain/operators/ep_dispatch.py:579-676, pithtrain/operators/all_to_all.py:19-47).
// All waits are bounded by PT_WAIT_LIMIT_NS and report through the status word.
#include "elementwise.cuh"
#include "host_common.h"
#include "ptx.cuh"
#include "peer_wait.cuh"

namespace pt {

constexpr int EP_MAX = 32;

struct EpChan {
  int ep, rank, cap, W, k;  // ranks, my rank, rows per source partition, row bytes, meta width
  long long off_data, off_mi, off_mf, off_count, off_flag, off_ack, off_done;
  unsigned char* base[EP_MAX];  // channel base on every rank (own entry included)
};

__device__ __forceinline__ unsigned char* chan_row(const EpChan& c, int peer, int slot, int src, int row) {
  return c.base[peer] + c.off_data + ((long long)(slot * c.ep + src) * c.cap + row) * c.W;
}
__device__ __forceinline__ int* chan_mi(const EpChan& c, int peer, int slot, int src, int row) {
  return reinterpret_cast<int*>(c.base[peer] + c.off_mi) + ((long long)(slot * c.ep + src) * c.cap + row) * c.k;
}
__device__ __forceinline__ float* chan_mf(const EpChan& c, int peer, int slot, int src, int row) {
  return reinterpret_cast<float*>(c.base[peer] + c.off_mf) + ((long long)(slot * c.ep + src) * c.cap + row) * c.k;
}
__device__ __forceinline__ int* chan_count(const EpChan& c, int peer, int slot, int src) {
  return reinterpret_cast<int*>(c.base[peer] + c.off_count) + slot * c.ep + src;
}
__device__ __forceinline__ unsigned* chan_flag(const EpChan& c, int peer, int slot, int src) {
  return reinterpret_cast<unsigned*>(c.base[peer] + c.off_flag) + slot * c.ep + src;
}
__device__ __forceinline__ unsigned* chan_ack(const EpChan& c, int peer, int slot, int dst) {
  return reinterpret_cast<unsigned*>(c.base[peer] + c.off_ack) + slot * c.ep + dst;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Spin until *p >= want (wrap-safe signed compare) or the time limit passes.
__device__ __forceinline__ bool wait_ge_bounded(const unsigned* p, unsigned want, int* err) {
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

// ----------------------------------------------------------------------------------------------
// Send-side plan: which tokens go to which rank, in token order (stable, no atomics).
// One CTA per destination rank.
// ----------------------------------------------------------------------------------------------
constexpr int PLAN_THREADS = 1024;

__global__ void __launch_bounds__(PLAN_THREADS)
ep_plan_kernel(const int* __restrict__ topk_idx, int m, int k, int experts_per_rank, int ep, int cap,
               int* __restrict__ token_send_pos, int* __restrict__ send_token_idx,
               int* __restrict__ send_eids, int* __restrict__ counts) {
  __shared__ int warp_tot[PLAN_THREADS / 32];
  const int d = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int running = 0;
  for (int start = 0; start < m; start += blockDim.x) {
    int t = start + threadIdx.x;
    bool hit = false;
    if (t < m) {
      for (int j = 0; j < k; ++j) hit |= (topk_idx[(size_t)t * k + j] / experts_per_rank == d);
    }
    unsigned bal = __ballot_sync(0xffffffffu, hit);
    int before = __popc(bal & ((1u << lane) - 1));
    if (lane == 0) warp_tot[w] = __popc(bal);
    __syncthreads();
    int woff = 0, tot = 0;
    for (int j = 0; j < nw; ++j) { int v = warp_tot[j]; if (j < w) woff += v; tot += v; }
    if (t < m) {
      int pos = running + woff + before;
      if (hit && pos < cap) {
        token_send_pos[(size_t)t * ep + d] = d * cap + pos;
        send_token_idx[(size_t)d * cap + pos] = t;
        for (int j = 0; j < k; ++j) {
          int e = topk_idx[(size_t)t * k + j];
          send_eids[((size_t)d * cap + pos) * k + j] = (e / experts_per_rank == d) ? e - d * experts_per_rank : -1;
        }
      } else {
        token_send_pos[(size_t)t * ep + d] = -1;
      }
    }
    running += tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[d] = min(running, cap);
}

// Wait until every peer acknowledged the previous use of `slot` (epoch - 2).
__global__ void ep_wait_acks_kernel(EpChan c, int slot, unsigned epoch, int* err) {
  int s = threadIdx.x;
  if (s < c.ep && epoch > 2) wait_ge_bounded(chan_ack(c, c.rank, slot, s), epoch - 2, err);
}

// Dispatch direction: gather rows by token index and store them into each destination's partition.
__global__ void __launch_bounds__(256)
ep_push_kernel(EpChan c, int slot, unsigned epoch, const unsigned char* __restrict__ src, long long src_stride,
               const int* __restrict__ send_token_idx, const int* __restrict__ counts,
               const int* __restrict__ send_eids, const float* __restrict__ weights, int* done, int* err) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int vec = c.W / 16;
  for (int d = 0; d < c.ep; ++d) {
    const int n = counts[d];
    if (!PT_IN_BOUNDS(n >= 0 && n <= c.cap, err)) continue;
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < n; r += gridDim.x * wpb) {
      const int t = send_token_idx[(size_t)d * c.cap + r];
      if (!PT_IN_BOUNDS(t >= 0 && t < c.cap, err)) continue;  // a partition holds at most one row per token
      const uint4* s4 = reinterpret_cast<const uint4*>(src + (size_t)t * src_stride);
      uint4* d4 = reinterpret_cast<uint4*>(chan_row(c, d, slot, c.rank, r));
      for (int v = lane; v < vec; v += 32) d4[v] = s4[v];
      if (c.k > 0 && lane < c.k) {
        chan_mi(c, d, slot, c.rank, r)[lane] = send_eids[((size_t)d * c.cap + r) * c.k + lane];
        chan_mf(c, d, slot, c.rank, r)[lane] = weights[(size_t)t * c.k + lane];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int prev = atomicAdd(done, 1);
    if (prev == (int)gridDim.x - 1) {
      *done = 0;
      __threadfence_system();
      for (int d = 0; d < c.ep; ++d) {
        *chan_count(c, d, slot, c.rank) = counts[d];
      }
      __threadfence_system();
      for (int d = 0; d < c.ep; ++d) st_release_sys(chan_flag(c, d, slot, c.rank), epoch);
    }
  }
}

// Receiver: wait for every source's flag, then prefix-sum the counts (prefix[ep+1], n_total).
__global__ void ep_wait_flags_kernel(EpChan c, int slot, unsigned epoch, int* prefix, int cap_total, int* err) {
  __shared__ int cnt[EP_MAX];
  int s = threadIdx.x;
  if (s < c.ep) {
    wait_ge_bounded(chan_flag(c, c.rank, slot, s), epoch, err);
    cnt[s] = prefix ? *chan_count(c, c.rank, slot, s) : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0 && prefix) {
    int acc = 0;
    for (int i = 0; i < c.ep; ++i) {
      prefix[i] = acc;
      int n = cnt[i];
      if (acc + n > cap_total) {
        n = cap_total - acc;
        if (err) atomicCAS(err, 0, PT_ERR_CAPACITY);
      }
      acc += n;
    }
    prefix[c.ep] = acc;
  }
}

// Compact the per-source partitions of my channel into dense outputs.
__global__ void __launch_bounds__(256)
ep_compact_kernel(EpChan c, int slot, const int* __restrict__ prefix, unsigned char* __restrict__ out_rows,
                  int* __restrict__ out_eids, float* __restrict__ out_w, int cap_total, int* err) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int total = prefix[c.ep];
  const int vec = c.W / 16;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < cap_total; i += gridDim.x * wpb) {
    if (i < total) {
      int s = 0;
      while (s + 1 < c.ep && prefix[s + 1] <= i) ++s;
      const int r = i - prefix[s];
      if (!PT_IN_BOUNDS(r >= 0 && r < c.cap, err)) continue;
      const uint4* s4 = reinterpret_cast<const uint4*>(chan_row(c, c.rank, slot, s, r));
      uint4* d4 = reinterpret_cast<uint4*>(out_rows + (size_t)i * c.W);
      for (int v = lane; v < vec; v += 32) d4[v] = s4[v];
      if (c.k > 0 && lane < c.k) {
        out_eids[(size_t)i * c.k + lane] = chan_mi(c, c.rank, slot, s, r)[lane];
        out_w[(size_t)i * c.k + lane] = chan_mf(c, c.rank, slot, s, r)[lane];
      }
    } else if (c.k > 0 && lane < c.k) {
      out_eids[(size_t)i * c.k + lane] = -1;
      out_w[(size_t)i * c.k + lane] = 0.f;
    }
  }
}

// Tell every source that `slot` of my channel has been consumed for `epoch`.
__global__ void ep_ack_kernel(EpChan c, int slot, unsigned epoch) {
  int s = threadIdx.x;
  if (s < c.ep) {
    __threadfence_system();
    st_release_sys(chan_ack(c, s, slot, c.rank), epoch);
  }
}

// Return direction: dense rows (compaction order) go back to the (my rank, position) cell of the
// rank they came from. `meta_f` optionally carries k floats per row (routing-weight gradients).
__global__ void __launch_bounds__(256)
ep_return_kernel(EpChan c, int slot, unsigned epoch, const unsigned char* __restrict__ rows,
                 const float* __restrict__ meta_f, const int* __restrict__ prefix, int* done, int* err) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int total = prefix[c.ep];
  const int vec = c.W / 16;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < total; i += gridDim.x * wpb) {
    int s = 0;
    while (s + 1 < c.ep && prefix[s + 1] <= i) ++s;
    const int r = i - prefix[s];
    if (!PT_IN_BOUNDS(r >= 0 && r < c.cap, err)) continue;  // the cell the row came from on rank s
    const uint4* s4 = reinterpret_cast<const uint4*>(rows + (size_t)i * c.W);
    uint4* d4 = reinterpret_cast<uint4*>(chan_row(c, s, slot, c.rank, r));
    for (int v = lane; v < vec; v += 32) d4[v] = s4[v];
    if (c.k > 0 && meta_f && lane < c.k) chan_mf(c, s, slot, c.rank, r)[lane] = meta_f[(size_t)i * c.k + lane];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int prev = atomicAdd(done, 1);
    if (prev == (int)gridDim.x - 1) {
      *done = 0;
      __threadfence_system();
      for (int d = 0; d < c.ep; ++d) st_release_sys(chan_flag(c, d, slot, c.rank), epoch);
    }
  }
}

}  // namespace pt

using namespace pt;

static inline int ep_grid(int cap_mult = 2) { return sm_count() * cap_mult; }

PT_API int pt_ep_chan_struct_size() { return (int)sizeof(EpChan); }

PT_API int pt_ep_plan(const int* topk_idx, int m, int k, int experts_per_rank, int ep, int cap,
                      int* token_send_pos, int* send_token_idx, int* send_eids, int* counts, void* stream_) {
  if (ep <= 0 || ep > EP_MAX || k > 32) return -1;
  ep_plan_kernel<<<ep, PLAN_THREADS, 0, (cudaStream_t)stream_>>>(topk_idx, m, k, experts_per_rank, ep, cap,
                                                                   token_send_pos, send_token_idx, send_eids, counts);
  return (int)cudaGetLastError();
}

// chan: pointer to a host copy of EpChan. done: device int (zero-initialised) private to the channel.
PT_API int pt_ep_push(const void* chan, int slot, unsigned epoch, const void* src, long long src_stride,
                      const int* send_token_idx, const int* counts, const int* send_eids, const float* weights,
                      int* done, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  EpChan c = *reinterpret_cast<const EpChan*>(chan);
  if (c.W % 16 != 0) return -1;
  int* err = device_status_word();
  ep_wait_acks_kernel<<<1, EP_MAX, 0, st>>>(c, slot, epoch, err);
  ep_push_kernel<<<ep_grid(), 256, 0, st>>>(c, slot, epoch, (const unsigned char*)src, src_stride, send_token_idx,
                                             counts, send_eids, weights, done, err);
  return (int)cudaGetLastError();
}

// Receiver side of a push: wait, prefix, compact into out_rows/out_eids/out_w, acknowledge.
PT_API int pt_ep_receive(const void* chan, int slot, unsigned epoch, int* prefix, void* out_rows, int* out_eids,
                         float* out_w, int cap_total, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  EpChan c = *reinterpret_cast<const EpChan*>(chan);
  int* err = device_status_word();
  ep_wait_flags_kernel<<<1, EP_MAX, 0, st>>>(c, slot, epoch, prefix, cap_total, err);
  ep_compact_kernel<<<ep_grid(), 256, 0, st>>>(c, slot, prefix, (unsigned char*)out_rows, out_eids, out_w, cap_total, err);
  ep_ack_kernel<<<1, EP_MAX, 0, st>>>(c, slot, epoch);
  return (int)cudaGetLastError();
}

PT_API int pt_ep_return(const void* chan, int slot, unsigned epoch, const void* rows, const float* meta_f,
                        const int* prefix, int* done, void* stream_) {
  cudaStream_t st = (cudaStream_t)stream_;
  EpChan c = *reinterpret_cast<const EpChan*>(chan);
  if (c.W % 16 != 0) return -1;
  int* err = device_status_word();
  ep_wait_acks_kernel<<<1, EP_MAX, 0, st>>>(c, slot, epoch, err);
  ep_return_kernel<<<ep_grid(), 256, 0, st>>>(c, slot, epoch, (const unsigned char*)rows, meta_f, prefix, done, err);
  return (int)cudaGetLastError();
}

// Home side of a return: wait for all flags (the reduction itself is the ordinary combine kernel
// reading the channel's data area), then acknowledge with pt_ep_ack once the data has been read.
PT_API int pt_ep_wait_returned(const void* chan, int slot, unsigned epoch, void* stream_) {
  EpChan c = *reinterpret_cast<const EpChan*>(chan);
  ep_wait_flags_kernel<<<1, EP_MAX, 0, (cudaStream_t)stream_>>>(c, slot, epoch, nullptr, 0, device_status_word());
  return (int)cudaGetLastError();
}

PT_API int pt_ep_ack(const void* chan, int slot, unsigned epoch, void* stream_) {
  EpChan c = *reinterpret_cast<const EpChan*>(chan);
  ep_ack_kernel<<<1, EP_MAX, 0, (cudaStream_t)stream_>>>(c, slot, epoch);
  return (int)cudaGetLastError();
}

// Sets this translation unit's copy of the peer-wait limit on the current device (see peer_wait.cuh).
extern "C" int pt_ep_set_wait_limit(unsigned long long ns) { return pt::set_peer_wait_limit_here(ns); }
