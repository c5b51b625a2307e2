"""Expert-order scatter and padded gather with the call signatures of the reference
(pithtrain/operators/token_scatter.py:26-35,328-367), for model code written against those helpers.

The framework's own expert block never materialises group sizes on the host: it sorts on the device into a statically
bounded layout (:func:`pithtrain_b200.ops.moe.route_sort`). ``scatter_for_grouped_gemm`` keeps the reference's
contract instead — an output of exactly ``grouped_mm_offs[-1]`` rows and the group sizes as a Python list — and
therefore reads the sizes back, as the reference does.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

__all__ = ["get_pinned_buffer", "scatter_for_grouped_gemm", "padded_index_gather"]

_PINNED: Dict[str, torch.Tensor] = {}


def get_pinned_buffer(name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
    """A reusable pinned host buffer of at least ``numel`` elements, keyed by ``name``."""
    buf = _PINNED.get(name)
    if buf is None or buf.numel() < numel or buf.dtype != dtype:
        buf = torch.empty(numel, dtype=dtype, pin_memory=torch.cuda.is_available())
        _PINNED[name] = buf
    return buf[:numel]


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dest, rows):
        out = x.new_zeros((rows, x.shape[1]))
        out.index_copy_(0, dest, x)
        ctx.save_for_backward(dest)
        return out

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        return g.index_select(0, dest), None, None


def scatter_for_grouped_gemm(input_tokens: torch.Tensor, expert_idxs: torch.Tensor, num_groups: int,
                             padding_alignment: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, List[int], torch.Tensor]:
    """Rows reordered by expert with every group zero-padded to ``padding_alignment`` rows.

    Returns ``(output_tokens [offs[-1], H], reverse_shuffle_idxs [m] int64, grouped_mm_offs [G] int32 cumulative padded
    ends, ks list[int], ks_tensor [G] int32)``; rows keep their input order inside a group.
    """
    m = input_tokens.shape[0]
    e = expert_idxs.long()
    counts = torch.bincount(e, minlength=num_groups)[:num_groups]
    padded = (counts + padding_alignment - 1) // padding_alignment * padding_alignment
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    order = torch.argsort(e, stable=True)
    first = torch.cumsum(counts, 0) - counts  # position of each group's first row in the sorted order
    sorted_e = e[order]
    pos = starts[sorted_e] + (torch.arange(m, device=e.device) - first[sorted_e])
    reverse = torch.empty(m, dtype=torch.int64, device=e.device)
    reverse[order] = pos
    ks_tensor = padded.to(torch.int32)
    ks = ks_tensor.tolist()  # host read-back: the reference's contract
    out = _Scatter.apply(input_tokens, reverse, int(sum(ks)))
    return out, reverse, ends.to(torch.int32), ks, ks_tensor


class _PaddedGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, index, pad):
        n = index.numel()
        buf = x.new_empty(((n + pad - 1) // pad * pad, ) + tuple(x.shape[1:]))
        out = buf[:n]
        torch.index_select(x, 0, index, out=out)
        ctx.save_for_backward(index)  # the input itself is not kept
        ctx.rows = x.shape[0]
        return out

    @staticmethod
    def backward(ctx, g):
        (index,) = ctx.saved_tensors
        gx = g.new_zeros((ctx.rows,) + tuple(g.shape[1:]))
        gx.index_add_(0, index, g)
        return gx, None, None


def padded_index_gather(input: torch.Tensor, index: torch.Tensor, pad_to_multiple: int = 1024) -> torch.Tensor:
    """``input[index]`` that does not keep ``input`` for the backward and rounds its allocation up to
    ``pad_to_multiple`` rows (stable allocator block sizes under varying counts)."""
    return _PaddedGather.apply(input, index.long(), pad_to_multiple)
