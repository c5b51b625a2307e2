"""Per-action memory trace of a training step, switched on without editing any code.

    PITHTRAIN_MEMORY_TRACE=0,3 torchrun ... script.py        # ranks 0 and 3 print one line per pipeline action

or, from Python, ``MemoryTrace(ranks={0}).attach(training.model)``. For every action of the DualPipeV schedule
(``F0``, ``FB(0,1)``, ``B1z``, ``W`` ...) the trace records the bytes allocated by the caching allocator, the bytes the
allocator holds beyond that, the device memory in use outside the allocator (CUDA context, NCCL, symmetric buffers),
and the bytes autograd kept for the backward during that action (distinct storages seen by a ``saved_tensors_hooks``
pack hook that hands tensors through unchanged). All of it is observation only: the order of operations does not
change; reading the allocator counters needs a device synchronize, so the traced step is slower.

The reference reaches the same view by having an agent patch print statements into six files
(.agents/skills/add-memory-prints/SKILL.md); here it is an observer on ``DualPipeV._run``.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Set

import torch
import torch.distributed as dist

GiB = float(1 << 30)


@dataclass
class TraceRow:
    index: int
    action: str
    allocated: int
    cached: int
    outside_allocator: int
    saved_for_backward: int
    peak_allocated: int

    def line(self) -> str:
        return (f"#{self.index:<4d}{self.action:<14s} alloc {self.allocated / GiB:8.3f}  cached {self.cached / GiB:7.3f}  "
                f"non-torch {self.outside_allocator / GiB:7.3f}  saved-by-autograd {self.saved_for_backward / GiB:+8.3f}  "
                f"peak {self.peak_allocated / GiB:8.3f}  GiB")


def device_memory() -> tuple:
    """``(allocated, cached, outside_allocator, peak_allocated)`` in bytes; zeros without a GPU."""
    if not torch.cuda.is_available():
        return 0, 0, 0, 0
    torch.cuda.synchronize()
    free, total = torch.cuda.mem_get_info()
    allocated, reserved = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    return allocated, reserved - allocated, max(0, total - free - reserved), torch.cuda.max_memory_allocated()


class SavedTensorBytes:
    """Context manager that sums the bytes of the distinct storages autograd saves while it is active."""

    def __init__(self) -> None:
        self.bytes = 0
        self._seen: Set[int] = set()
        self._hooks = None

    def _pack(self, t: torch.Tensor) -> torch.Tensor:
        try:
            st = t.untyped_storage()
            key = st.data_ptr()
            if key and key not in self._seen:
                self._seen.add(key)
                self.bytes += st.nbytes()
        except Exception:  # tensors without storage (meta, fake) carry no memory
            pass
        return t

    def __enter__(self) -> "SavedTensorBytes":
        self._hooks = torch.autograd.graph.saved_tensors_hooks(self._pack, lambda t: t)
        self._hooks.__enter__()
        return self

    def __exit__(self, *exc) -> None:
        self._hooks.__exit__(*exc)
        self._hooks = None


class MemoryTrace:
    """Observer of a ``DualPipeV``: one :class:`TraceRow` per executed action, printed on the chosen ranks."""

    def __init__(self, ranks: Optional[Iterable[int]] = (0,), sink: Optional[Callable[[str], None]] = print) -> None:
        self.ranks = None if ranks is None else set(ranks)
        self.sink = sink
        self.rows: List[TraceRow] = []
        self._pipe = None
        self._orig = None

    def _active(self) -> bool:
        r = dist.get_rank() if dist.is_initialized() else 0
        return self.ranks is None or r in self.ranks

    def attach(self, pipe) -> "MemoryTrace":
        assert self._pipe is None, "already attached"
        self._pipe, self._orig = pipe, pipe._run
        if not self._active():
            return self
        rank = dist.get_rank() if dist.is_initialized() else 0

        def traced(action):
            with SavedTensorBytes() as saved:
                self._orig(action)
            a, c, o, p = device_memory()
            row = TraceRow(len(self.rows), repr(action), a, c, o, saved.bytes, p)
            self.rows.append(row)
            if self.sink is not None:
                self.sink(f"[memory rank {rank}] {row.line()}")

        pipe._run = traced
        return self

    def detach(self) -> None:
        if self._pipe is not None:
            self._pipe._run = self._orig
        self._pipe = self._orig = None

    def reset(self) -> None:
        self.rows.clear()

    def peak(self) -> Optional[TraceRow]:
        return max(self.rows, key=lambda r: r.allocated, default=None)


def ranks_from_env(value: Optional[str] = None) -> Optional[Set[int]]:
    """``"0,3"`` -> ``{0, 3}``; ``"all"`` -> every rank (``None``); unset or empty -> no tracing (empty set)."""
    v = os.environ.get("PITHTRAIN_MEMORY_TRACE", "") if value is None else value
    v = v.strip()
    if not v:
        return set()
    if v == "all":
        return None
    return {int(x) for x in v.split(",") if x.strip()}


def attach_from_env(pipe) -> Optional[MemoryTrace]:
    """Called by ``setup_training``: attaches a trace when ``PITHTRAIN_MEMORY_TRACE`` names ranks."""
    ranks = ranks_from_env()
    if ranks is not None and not ranks:
        return None
    return MemoryTrace(ranks=ranks).attach(pipe)
