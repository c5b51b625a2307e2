"""Grouped (per-expert) linear layers over expert-sorted rows.

Rows of the input are grouped by expert with device-side offsets ``offs[E+1]`` (groups aligned to 16
rows, see :func:`pithtrain_b200.ops.moe.route_sort`). Forward and dgrad are M-grouped GEMMs, the
weight gradient is a K-grouped GEMM that accumulates into the ``[E, out, in]`` gradient buffer in
its epilogue and can be deferred through ``WeightGradStore``. Nothing is read back to the host.
Reference counterpart: pithtrain/operators/grouped_linear.py:18-85.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..dualpipe.utils import WeightGradStore
from . import gemm as G
from .common import grad_buffer


class _GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offs, grad_getter, save_input):
        y = G.grouped_gemm_nt(x, w, offs)
        ctx.save_for_backward(x if save_input else None, w, offs)
        ctx.grad_getter = grad_getter
        ctx.x_provider = None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, offs = ctx.saved_tensors
        dy = dy.contiguous()
        dx = G.grouped_gemm_nn(dy, w, offs) if ctx.needs_input_grad[0] else None
        get = ctx.grad_getter

        def wgrad_fn(dy=dy, x=x, offs=offs):
            G.grouped_gemm_tn(dy, x, offs, get(), accumulate=True)

        if WeightGradStore.enabled:
            WeightGradStore.put(wgrad_fn)
        else:
            wgrad_fn()
        return dx, None, None, None, None


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, offs: torch.Tensor,
                   weight_param: Optional[torch.Tensor] = None, grad_getter=None, fp8: Optional[bool] = None) -> torch.Tensor:
    """``y[rows of group g] = x[rows of group g] @ weight[g].T`` for ``weight[E, out, in]``."""
    wp = weight if weight_param is None else weight_param
    if grad_getter is None:
        grad_getter = lambda: grad_buffer(wp)  # noqa: E731
    if not x.requires_grad and torch.is_grad_enabled():
        x = x.detach().requires_grad_()
    from . import fp8_linear

    if fp8_linear.eligible(x, weight, fp8):
        return fp8_linear.fp8_grouped_linear_apply(x, weight, offs, grad_getter)
    return _GroupedLinearFn.apply(x, weight, offs, grad_getter, True)


class GroupedLinear(nn.Module):
    """``num_groups`` independent ``in_features -> out_features`` projections stored as one
    ``[E, out, in]`` parameter (the in-memory expert layout of the reference)."""

    def __init__(self, num_groups: int, in_features: int, out_features: int, device=None, dtype=None):
        super().__init__()
        self.num_groups, self.in_features, self.out_features = num_groups, in_features, out_features
        self.weight = nn.Parameter(torch.empty((num_groups, out_features, in_features), device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=0.02)

    fp8: Optional[bool] = None

    def forward(self, x: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
        return grouped_linear(x, self.weight, offs, fp8=self.fp8)

    def extra_repr(self) -> str:
        return f"groups={self.num_groups}, in={self.in_features}, out={self.out_features}"


def __getattr__(name: str):
    # ``FP8GroupedLinear`` lives with the fp8 path; the reference exports it from this module
    # (pithtrain/operators/grouped_linear.py:239), so it resolves here too, lazily to keep the imports acyclic.
    if name == "FP8GroupedLinear":
        from .fp8_linear import FP8GroupedLinear

        return FP8GroupedLinear
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
