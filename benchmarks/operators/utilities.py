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
