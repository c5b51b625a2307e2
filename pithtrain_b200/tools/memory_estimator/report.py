"""Text report of an :class:`Estimate` (summary, per-tensor detail, schedule timeline, verdict)."""

from __future__ import annotations

from typing import List

from .activation_profile import layer_saved
from .model_profile import ModelDims, ParallelCfg, chunk_layers
from .schedule_simulator import Estimate

GiB = 1024 ** 3


def fmt(n: float) -> str:
    for unit, div in (("GiB", GiB), ("MiB", 1024 ** 2), ("KiB", 1024)):
        if abs(n) >= div:
            return f"{n / div:8.2f} {unit}"
    return f"{n:8.0f} B  "


def verdict(peak: int, gpu_gb: float) -> str:
    cap = gpu_gb * 1e9
    if peak > cap:
        return "OOM"
    return "TIGHT" if peak > 0.92 * cap else "OK"


def summary_lines(est: Estimate, dims: ModelDims, par: ParallelCfg, pp_rank: int, gpu_gb: float) -> List[str]:
    out = [f"model {dims.model_type}: {dims.L} layers, hidden {dims.H}, {dims.E} experts top-{dims.k}, vocab {dims.V}",
           f"mesh pp={par.pp} dp={par.dp} cp={par.cp} ep={par.ep} ({par.world} GPUs), pp_rank={pp_rank}; "
           f"micro-batch {par.micro_batch_size}×{par.sequence_length}, global batch {par.global_batch_size}, "
           f"{par.num_chunks} micro-batches per step",
           f"tokens per micro-batch {est.tokens.T}; expert rows received {est.tokens.recv} (buffers hold "
           f"{est.tokens.recv_capacity}); sorted rows {est.tokens.sorted_rows}",
           f"micro-batches in flight at most: chunk0 {est.max_inflight[0]}, chunk1 {est.max_inflight[1]}; "
           f"one micro-batch holds {fmt(est.chunk_bytes[0]).strip()} / {fmt(est.chunk_bytes[1]).strip()}", ""]
    for name, b in est.categories().items():
        if b or not name.startswith("fp8"):
            out.append(f"  {name:<52s}{fmt(b)}")
    out.append(f"  {'-' * 52}{'-' * 12}")
    out.append(f"  {'estimated peak (at ' + est.peak_event.action + ', action #' + str(est.peak_event.step) + ')':<52s}{fmt(est.peak_total)}")
    if est.static.optimizer_host:
        out.append(f"  {'optimizer state in pinned host memory':<52s}{fmt(est.static.optimizer_host)}")
    out.append(f"  device capacity {gpu_gb:.0f} GB -> {verdict(est.peak_total, gpu_gb)}")
    return out


def detail_lines(dims: ModelDims, par: ParallelCfg, pp_rank: int, est: Estimate) -> List[str]:
    out = []
    for phase, layers in enumerate(chunk_layers(dims, par, pp_rank)):
        if not len(layers):
            continue
        idx = layers[len(layers) // 2]
        out.append(f"chunk {phase}: layers {layers.start}..{layers.stop - 1}; tensors kept by layer {idx} for one micro-batch")
        for s in sorted(layer_saved(dims, par, idx, est.tokens), key=lambda s: -s.nbytes):
            if s.nbytes:
                out.append(f"    stage {s.stage}  {s.name:<24s}{fmt(s.nbytes)}{'   (kept for deferred wgrad)' if s.wgrad else ''}")
    return out


def timeline_lines(est: Estimate, limit: int) -> List[str]:
    ev = est.timeline if limit <= 0 else est.timeline[:limit]
    out = [f"{'#':>5s}  {'action':<14s}{'activations':>14s}{'wgrad store':>14s}{'total':>14s}"]
    for e in ev:
        out.append(f"{e.step:5d}  {e.action:<14s}{fmt(e.live_activations):>14s}{fmt(e.wgrad_store):>14s}{fmt(e.total):>14s}")
    if limit > 0 and len(est.timeline) > limit:
        out.append(f"... {len(est.timeline) - limit} more actions")
    return out


def suggestion_lines(est: Estimate, par: ParallelCfg, gpu_gb: float) -> List[str]:
    if verdict(est.peak_total, gpu_gb) == "OK":
        return []
    out = ["ways to lower the peak:"]
    if not par.offload_optimizer_state and est.static.optimizer_device > 4 * GiB:
        out.append(f"  - offload_optimizer_state=True moves {fmt(est.static.optimizer_device).strip()} to pinned host memory")
    if par.grad_dtype == "fp32":
        out.append(f"  - grad_dtype='bf16' halves the gradient accumulators ({fmt(est.static.grads // 2).strip()} saved)")
    out.append("  - a larger expert- or pipeline-parallel size divides parameters and gradients")
    if par.micro_batch_size > 1:
        out.append("  - micro_batch_size=1 shrinks every in-flight activation set")
    return out
