"""Engine utilities: deferred weight-gradient store, quantised-weight cache versioning, manual
backward driver, micro-batch scatter/gather and memory printers.

``WeightGradStore`` is what makes the zero-bubble W phases possible: linear layers hand their
weight-gradient GEMM to the store as a closure when it is enabled, and the scheduler runs the
closures later, in FIFO order of the backward chunks that produced them
(the behaviour of pithtrain/dualpipe/utils.py:24-132 in the reference).
"""

from __future__ import annotations

from collections import deque
from typing import Callable, List, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn


class FP8WeightCacheControl:
    """Version counter for per-step caches of quantised weights.

    Weights are constant across the micro-batches of one ``DualPipeV.step``; modules tag their
    cached fp8 copies with ``version`` and re-quantise when it changes.
    """

    version: int = 0
    caches: List[dict] = []  # module-level caches registered by the fp8 operators

    @classmethod
    def step(cls) -> None:
        cls.version += 1

    @classmethod
    def clear(cls, *modules: nn.Module) -> None:
        for module in modules:
            for m in module.modules():
                if hasattr(m, "_wq_cache"):
                    m._wq_cache = None
        for cache in cls.caches:
            cache.clear()


class WeightGradStore:
    enabled: bool = False
    cache: List[Callable] = []
    funcs_queue: deque = deque()

    @classmethod
    def put(cls, func: Callable) -> None:
        cls.cache.append(func)

    @classmethod
    def flush(cls) -> None:
        cls.funcs_queue.append(cls.cache)
        cls.cache = []

    @classmethod
    def pop(cls) -> None:
        assert cls.funcs_queue, "WeightGradStore.pop on an empty queue"
        with torch.no_grad():
            for func in cls.funcs_queue.popleft():
                func()

    @classmethod
    def clear(cls) -> None:
        cls.cache = []
        cls.funcs_queue = deque()


def run_backward(tensors: Sequence[torch.Tensor | None], grad_tensors: Sequence[torch.Tensor | None]) -> None:
    """Backward from several roots at once, skipping ``None`` entries and grad-less tensors."""
    pairs = [(t, g) for t, g in zip(tensors, grad_tensors) if t is not None and t.requires_grad]
    if not pairs:
        return
    ts, gs = zip(*pairs)
    with torch.autograd.set_multithreading_enabled(False):
        torch.autograd.backward(ts, gs)


def chunk_tensor(x, chunks: int, dim: int):
    if x is None:
        return [None] * chunks
    return x.tensor_split(chunks, dim=dim)


def cat_tensor(xs, dim: int):
    if isinstance(xs, (tuple, list)):
        if xs[0] is None:
            assert all(y is None for y in xs)
            return None
        if len(xs) == 1:
            return xs[0]
    return torch.cat(xs, dim=dim)


def scatter(inputs, chunks: int, dim: int):
    """Split a tensor (or tuple of tensors) into ``chunks`` micro-batches along ``dim``."""
    if isinstance(inputs, torch.Tensor):
        inputs = (inputs,)
    cols = [chunk_tensor(x, chunks, dim) for x in inputs]
    micro = list(zip(*cols))
    return micro if micro else [() for _ in range(chunks)]


def gather(micro_outputs, dim: int):
    if isinstance(micro_outputs[0], torch.Tensor):
        micro_outputs = [(x,) for x in micro_outputs]
    return tuple(cat_tensor(list(col), dim=dim) for col in zip(*micro_outputs))


def free_storage(*tensors: torch.Tensor | None) -> None:
    """Release the memory behind tensors whose values are dead but whose objects are still referenced."""
    for t in tensors:
        if t is not None and t.untyped_storage().size() > 0 and t._base is None:
            t.untyped_storage().resize_(0)


def format_size(n: float) -> str:
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if abs(n) < 1024 or unit == "TiB":
            return f"{n:.2f} {unit}"
        n /= 1024
    return f"{n:.2f} TiB"


def print_msg(msg: str, rank: int | None = 0) -> None:
    r = dist.get_rank() if dist.is_initialized() else 0
    if rank is None or r == rank:
        print(f"[rank {r}] {msg}", flush=True)


def print_model_size_grad_size_per_device(model: nn.Module, rank: int | None = 0) -> None:
    p = sum(x.numel() * x.element_size() for x in model.parameters())
    g = sum(x.grad.numel() * x.grad.element_size() for x in model.parameters() if x.grad is not None)
    print_msg(f"parameters {format_size(p)}  gradients {format_size(g)}", rank)


def print_memory(tag: str, rank: int | None = 0) -> None:
    if torch.cuda.is_available():
        a, r, m = torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.max_memory_allocated()
        print_msg(f"{tag}: allocated {format_size(a)} reserved {format_size(r)} peak {format_size(m)}", rank)
