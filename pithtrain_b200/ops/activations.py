"""Gated activations as autograd ops: SwiGLU on a packed ``[rows, 2I]`` tensor, ``silu_mul`` on two
tensors, the GPT-OSS clamped SwiGLU on interleaved columns, and ``indexed_bias_add`` with a
segmented-sum backward. Reference counterparts: pithtrain/operators/silu_mul.py,
pithtrain/operators/clamped_swiglu.py, pithtrain/operators/indexed_bias_add.py.
"""

from __future__ import annotations

import torch

from .common import accumulate_grad
from .moe import indexed_bias_add_rows, segment_sum, swiglu_bwd, swiglu_fwd


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, interleaved, alpha, limit):
        shape = gu.shape
        gu2 = gu.reshape(-1, shape[-1]).contiguous()
        ctx.save_for_backward(gu2)
        ctx.cfg = (interleaved, alpha, limit, shape)
        return swiglu_fwd(gu2, None, interleaved, alpha, limit).view(*shape[:-1], shape[-1] // 2)

    @staticmethod
    def backward(ctx, dact):
        (gu2,) = ctx.saved_tensors
        interleaved, alpha, limit, shape = ctx.cfg
        dgu, _, _ = swiglu_bwd(gu2, dact.reshape(-1, shape[-1] // 2), None, None, interleaved, alpha, limit)
        return dgu.view(shape), None, None, None


def swiglu(gu: torch.Tensor, interleaved: bool = False, alpha: float = 1.0, limit: float = 0.0) -> torch.Tensor:
    """``silu(gate) * up`` on packed ``[.., 2I]`` (gate columns first, or interleaved gate/up)."""
    return _SwiGLUFn.apply(gu, interleaved, alpha, limit)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up``; backward recomputes the sigmoid and saves only gate/up."""
    return swiglu(torch.cat([gate, up], dim=-1))


def clamped_swiglu(gate_up: torch.Tensor, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """GPT-OSS activation on interleaved ``[.., 2N]``: ``(clamp(u,±L)+1) * min(g,L) * sigmoid(alpha*min(g,L))``."""
    return swiglu(gate_up, interleaved=True, alpha=alpha, limit=limit)


class _IndexedBiasAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, offs):
        ctx.save_for_backward(offs)
        ctx.bias_ref = bias
        return indexed_bias_add_rows(x, bias.detach(), offs)

    @staticmethod
    def backward(ctx, dy):
        (offs,) = ctx.saved_tensors
        b = ctx.bias_ref
        accumulate_grad(b, segment_sum(dy, offs, b.shape[0]))
        return dy, None, None


def indexed_bias_add(x: torch.Tensor, bias: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """``x[r] + bias[group(r)]`` for rows grouped by ``offs``; the bias gradient is a per-group row sum."""
    return _IndexedBiasAddFn.apply(x, bias, offs)
