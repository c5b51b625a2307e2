"""Asynchronous ``all_to_all_single`` without autograd, as the reference exposes it
(pithtrain/operators/all_to_all.py:20-47): the returned tensor carries the ``Work`` handle as ``.comm_work`` and the
caller waits on it and writes the backward itself. The framework's own expert exchange does not go through this
function (see :mod:`pithtrain_b200.parallel.ep`); it exists for model code written against the reference's helpers."""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

__all__ = ["direct_all_to_all"]

_PAD_ROWS = 1024  # allocations are rounded up so that varying receive counts reuse the same allocator blocks


def direct_all_to_all(input: torch.Tensor, output_split_sizes: List[int], input_split_sizes: List[int],
                      group: dist.ProcessGroup) -> torch.Tensor:
    n = sum(output_split_sizes)
    buf = input.new_empty(((n + _PAD_ROWS - 1) // _PAD_ROWS * _PAD_ROWS,) + tuple(input.shape[1:]))
    out = buf[:n]
    out.comm_work = dist.all_to_all_single(out, input.contiguous(), output_split_sizes, input_split_sizes, group=group,
                                           async_op=True)
    return out
