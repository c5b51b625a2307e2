"""Fused cross-entropy: one kernel computes per-token losses and overwrites the logits with their
gradient; backward only scales that buffer by the incoming gradient.

``cross_entropy(logits[n,V], labels[n], reduction="sum")`` returns the summed loss over
non-ignored tokens (the criterion of the training task multiplies nothing else in). Because the
logits buffer is reused for the gradient, the caller must not use ``logits`` afterwards — the same
contract as pithtrain/operators/cross_entropy.py:82-125.
"""

from __future__ import annotations

import torch

from .. import _native
from .common import sp, use_native


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        n, V = logits.shape
        assert logits.is_contiguous() or logits.stride(1) == 1
        loss = torch.empty(n, dtype=torch.float32, device=logits.device)
        rc = _native.lib().pt_cross_entropy(logits.data_ptr(), labels.contiguous().data_ptr(), loss.data_ptr(), n, V,
                                            logits.stride(0), int(ignore_index), sp())
        _native.check(rc, "pt_cross_entropy")
        # the kernel wrote through the raw pointer, so autograd's version counter is untouched
        ctx.save_for_backward(logits)
        return loss.sum()

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        if grad.is_contiguous() and grad.numel() % 8 == 0:
            gs = g.reshape(1).float().contiguous()
            rc = _native.lib().pt_scale_bf16(grad.data_ptr(), gs.data_ptr(), grad.numel(), sp())
            _native.check(rc, "pt_scale_bf16")
        else:
            grad.mul_(g.to(grad.dtype))
        return grad, None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                  reduction: str = "sum") -> torch.Tensor:
    V = logits.shape[-1]
    lg = logits.reshape(-1, V)
    lb = labels.reshape(-1)
    if use_native(lg) and lg.stride(0) % 8 == 0 and lg.stride(1) == 1 and lb.dtype == torch.int64:
        if not lg.requires_grad and not torch.is_grad_enabled():
            lg = lg.clone()
        loss = _CrossEntropyFn.apply(lg, lb, ignore_index)
    else:
        loss = torch.nn.functional.cross_entropy(lg.float(), lb, ignore_index=ignore_index, reduction="sum")
    if reduction == "mean":
        loss = loss / (lb != ignore_index).sum().clamp(min=1)
    return loss
