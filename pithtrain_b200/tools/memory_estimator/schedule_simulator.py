"""Replay one rank's DualPipeV action list and track live device memory.

The action list is the same data the executor runs (pithtrain_b200/dualpipe/schedule.py), so the
estimator cannot drift from the engine: ``F`` allocates one micro-batch's activations for a chunk,
``B`` releases them (keeping what the deferred weight gradients need when the action is a
zero-bubble ``B``), ``W`` releases the oldest deferred set, ``FB`` holds both at once. The reference
re-implements its eight phases for the same purpose (tools/memory_estimator/schedule_simulator.py:93-346
of the reference).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Tuple

from ...dualpipe.schedule import build_schedule
from .activation_profile import TokenCounts, edge_bytes, layer_bytes, token_counts
from .model_profile import ModelDims, ParallelCfg, StaticMemory, chunk_layers, static_memory

GiB = 1024 ** 3


@dataclass
class Event:
    step: int
    action: str
    live_activations: int
    wgrad_store: int
    total: int


@dataclass
class Estimate:
    static: StaticMemory
    tokens: TokenCounts
    chunk_bytes: Tuple[int, int]
    chunk_wgrad_bytes: Tuple[int, int]
    transient: int
    comm_buffers: int
    runtime_overhead: int
    peak_activations: int
    peak_total: int
    peak_event: Event
    timeline: List[Event] = field(default_factory=list)
    max_inflight: Tuple[int, int] = (0, 0)

    def categories(self) -> Dict[str, int]:
        return {"parameters": self.static.params, "gradient accumulators": self.static.grads,
                "optimizer state (device)": self.static.optimizer_device,
                "fp8 weight copies (both orientations)": self.static.fp8_weights,
                "activations + deferred wgrad at peak": self.peak_activations, "transient workspace": self.transient,
                "communication buffers": self.comm_buffers, "runtime (context, NCCL, cuBLAS/cuDNN workspaces)": self.runtime_overhead}


def runtime_overhead_bytes(par: ParallelCfg) -> int:
    """Memory outside the caching allocator: CUDA context + library handles (~0.6 GiB), one NCCL
    communicator per active mesh axis (~0.35 GiB each incl. the world group), cuBLAS/cuDNN
    workspaces (~0.5 GiB)."""
    axes = 1 + sum(x > 1 for x in (par.pp, par.ep, par.dp, par.cp))
    return int((0.6 + 0.35 * axes + 0.5) * GiB) if par.world > 1 else int(1.1 * GiB)


def comm_buffer_bytes(dims: ModelDims, par: ParallelCfg, tc: TokenCounts) -> int:
    n = 0
    if par.ep > 1 and par.ep_backend == "fused":
        # four channels (dispatch/combine × forward/backward), two slots, ep partitions of T rows
        cells = 2 * par.ep * tc.T
        n += 4 * cells * dims.H * 2 + 2 * cells * dims.k * 8
    if par.pp > 1:
        n += 4 * tc.T * dims.H * 2  # activations / gradients in flight in each direction
    if par.cp > 1:
        # context-parallel payload exchange (one per payload shape, shared by all layers): two slots of the published
        # K/V (or MLA latent + rope key) in bf16, and two slots of cp per-writer gradient partitions in fp32
        per_token = (dims.kv_lora + dims.d_rope) if dims.kv_lora else dims.nkv * (dims.d_qk + dims.d_v)
        n += 2 * tc.T * per_token * 2 + 2 * par.cp * tc.T * per_token * 4
    return n


def estimate(dims: ModelDims, par: ParallelCfg, pp_rank: int = 0, imbalance: float = 1.0, fragmentation: float = 0.05,
             keep_timeline: bool = False) -> Estimate:
    tc = token_counts(dims, par, imbalance)
    static = static_memory(dims, par, pp_rank)
    chunks = chunk_layers(dims, par, pp_rank)
    S = 2 * par.pp
    per_chunk, per_chunk_w, biggest_layer = [], [], 0
    for phase, layers in enumerate(chunks):
        tot = held = 0
        for idx in layers:
            a, w = layer_bytes(dims, par, idx, tc)
            tot, held, biggest_layer = tot + a, held + w, max(biggest_layer, a)
        stage = pp_rank if phase == 0 else S - 1 - pp_rank
        tot += edge_bytes(dims, par, first=(stage == 0), last=(stage == S - 1), tc=tc)
        per_chunk.append(tot)
        per_chunk_w.append(held)
    # backward of one layer materialises gradients of about everything that layer saved
    transient = int(1.5 * biggest_layer)
    live = [0, 0]
    peak_inflight = [0, 0]
    store: Deque[int] = deque()
    timeline: List[Event] = []
    peak = Event(0, "-", 0, 0, 0)
    base = static.device_total + comm_buffer_bytes(dims, par, tc) + runtime_overhead_bytes(par) + transient

    def snapshot(step: int, name: str, extra: int = 0) -> None:
        nonlocal peak
        acts = live[0] * per_chunk[0] + live[1] * per_chunk[1] + extra
        ev = Event(step, name, acts, sum(store), base + acts + sum(store))
        if keep_timeline:
            timeline.append(ev)
        if ev.total > peak.total:
            peak = ev

    for step, a in enumerate(build_schedule(par.pp, pp_rank, max(par.num_chunks, 2 * par.pp))):
        if a.kind == "F":
            live[a.phase] += 1
            snapshot(step, repr(a))
        elif a.kind == "B":
            snapshot(step, repr(a))
            live[a.phase] -= 1
            if a.zb:
                store.append(per_chunk_w[a.phase])
        elif a.kind == "FB":
            live[a.phase] += 1
            snapshot(step, repr(a))
            live[a.bphase] -= 1
        elif a.kind == "W":
            snapshot(step, repr(a))
            if store:
                store.popleft()
        for p in (0, 1):
            peak_inflight[p] = max(peak_inflight[p], live[p])
    assert live == [0, 0] and not store, "schedule left activations alive"
    frag = int(fragmentation * (peak.live_activations + peak.wgrad_store + transient))
    return Estimate(static=static, tokens=tc, chunk_bytes=tuple(per_chunk), chunk_wgrad_bytes=tuple(per_chunk_w),
                    transient=transient + frag, comm_buffers=comm_buffer_bytes(dims, par, tc),
                    runtime_overhead=runtime_overhead_bytes(par), peak_activations=peak.live_activations + peak.wgrad_store,
                    peak_total=peak.total + frag, peak_event=peak, timeline=timeline, max_inflight=tuple(peak_inflight))
