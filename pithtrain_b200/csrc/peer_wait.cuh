// Time limit of waits on another GPU's flag (system-scope spins in the expert-parallel, shard-group and
// context-parallel transports). A run-time value, so that production jobs can use a long, still bounded, limit
// (a rank may legitimately stall for seconds in data loading or lazy initialisation) while tests keep it short.
// The variable is per translation unit (the library is not built with relocatable device code); the host entry
// point pt_set_peer_wait_limit_ns updates every copy on the current device.
#pragma once
#include <cuda_runtime.h>
#include "ptx.cuh"

namespace pt {
static __device__ unsigned long long pt_peer_wait_limit_ns = PT_WAIT_LIMIT_NS;

static inline int set_peer_wait_limit_here(unsigned long long ns) {
  return cudaMemcpyToSymbol(pt_peer_wait_limit_ns, &ns, sizeof(ns)) == cudaSuccess ? 0 : -1;
}
}  // namespace pt
