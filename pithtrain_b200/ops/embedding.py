"""Token embedding lookup whose backward accumulates into the parameter's gradient buffer."""

from __future__ import annotations

import torch

from .common import grad_buffer
from .moe import gather_rows


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        ctx.save_for_backward(ids)
        ctx.w_ref = weight
        flat = ids.reshape(-1)
        if weight.is_cuda and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0:
            out = gather_rows(weight.detach(), flat.int().contiguous())
        else:
            out = weight.detach()[flat]
        return out.view(*ids.shape, weight.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.w_ref
        g = grad_buffer(w)
        g.index_add_(0, ids.reshape(-1), dy.reshape(-1, dy.shape[-1]).to(g.dtype))
        return None, None


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    out = _EmbeddingFn.apply(ids, weight)
    return out


class Embedding(torch.nn.Embedding):
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if torch.is_grad_enabled() and self.weight.requires_grad:
            # route through autograd with a dummy edge so backward() runs
            return _EmbeddingFn.apply(ids, self.weight)
        return _EmbeddingFn.apply(ids, self.weight)
