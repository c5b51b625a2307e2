"""Timing helper shared by the operator benchmarks: CUDA events, warm-up, L2 flush between iterations."""

import json
from pathlib import Path

import torch

_FLUSH = None


def peaks() -> dict:
    """Measured roofline denominators of this pool if the file is present, else an earlier measurement."""
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        return json.load(open(p))
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


def bench(fn, iters: int = 20, warmup: int = 5) -> float:
    """Median milliseconds of ``fn()``; a 256 MiB buffer is rewritten before every timed call to evict L2."""
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        _FLUSH.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def rand_bf16(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).bfloat16()


def make_routing(tokens: int, experts: int, k: int, kind: str = "uniform", seed: int = 0, zipf_a: float = 1.2) -> torch.Tensor:
    """``[tokens, k]`` int32 expert ids on the CPU, ``k`` distinct experts per token.

    ``uniform``: every subset equally likely. ``normal``: top-k of router logits drawn from N(0, 1) (near-uniform load).
    ``zipf``: expert ``e`` is picked with probability proportional to ``1 / (e + 1) ** zipf_a`` without replacement
    (Gumbel top-k), so the first ranks of an expert-parallel group receive most of the traffic.
    """
    g = torch.Generator().manual_seed(seed)
    if kind == "uniform":
        return torch.rand(tokens, experts, generator=g).topk(k, dim=-1).indices.int()
    if kind == "normal":
        return torch.randn(tokens, experts, generator=g).topk(k, dim=-1).indices.int()
    if kind == "zipf":
        logp = -zipf_a * torch.log(torch.arange(1, experts + 1, dtype=torch.float32))
        u = torch.rand(tokens, experts, generator=g).clamp_(1e-12, 1 - 1e-7)
        return (logp - torch.log(-torch.log(u))).topk(k, dim=-1).indices.int()
    raise ValueError(f"unknown routing {kind!r}")


def remote_rows_by_destination(idx: torch.Tensor, experts: int, ep: int, rank: int) -> torch.Tensor:
    """``[ep]`` int64: de-duplicated rows that source rank ``rank`` stores into each other GPU for routing ``idx``."""
    dest = idx.long() // (experts // ep)
    hit = torch.zeros(idx.shape[0], ep, dtype=torch.bool).scatter_(1, dest, True)
    hit[:, rank] = False
    return hit.sum(0)
