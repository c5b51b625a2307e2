"""Router top-k with its softmax, forward and backward, in one kernel each.

* ``mode="softmax_topk"``: ``p = softmax(logits)`` in fp32, top-k of ``p``, optional renormalisation,
  times ``scale`` (Qwen3-MoE, DeepSeek-V2: pithtrain/models/qwen3_moe.py:81-89,
  pithtrain/models/deepseek_v2.py:149-164).
* ``mode="topk_softmax"``: top-k of the logits, softmax over the picked k (GPT-OSS:
  pithtrain/models/gpt_oss.py:176-182).

Returns ``(topk_weight[n,k] fp32, topk_idx[n,k] int32, probs[n,E] fp32 or None)``. ``probs`` is a
differentiable output so a load-balance loss can be built on it with ordinary autograd; its
gradient is folded into the same backward kernel.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native
from .common import sp

MODES = {"softmax_topk": 0, "topk_softmax": 1}


def router_topk_ref(logits, k, mode="softmax_topk", renorm=False, scale=1.0):
    lf = logits.float()
    if mode == "softmax_topk":
        p = lf.softmax(-1)
        w, idx = torch.topk(p, k, dim=-1)
        if renorm:
            w = w / w.sum(-1, keepdim=True)
        return w * scale, idx.int(), p
    v, idx = torch.topk(lf, k, dim=-1)
    return v.softmax(-1) * scale, idx.int(), None


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, mode, renorm, scale):
        n, E = logits.shape
        L = _native.lib()
        lg = logits.contiguous()
        probs = torch.empty((n, E), dtype=torch.float32, device=lg.device) if mode == 0 else None
        idx = torch.empty((n, k), dtype=torch.int32, device=lg.device)
        w = torch.empty((n, k), dtype=torch.float32, device=lg.device)
        rc = L.pt_router_topk_fwd(lg.data_ptr(), int(lg.dtype == torch.float32), None if probs is None else probs.data_ptr(),
                                  idx.data_ptr(), w.data_ptr(), n, E, k, mode, int(renorm), float(scale), sp())
        _native.check(rc, "pt_router_topk_fwd")
        ctx.save_for_backward(probs, idx, w)
        ctx.cfg = (k, mode, renorm, scale, lg.dtype)
        ctx.mark_non_differentiable(idx)
        if probs is None:
            return w, idx
        return w, idx, probs

    @staticmethod
    def backward(ctx, dw, didx=None, dprobs=None):
        probs, idx, w = ctx.saved_tensors
        k, mode, renorm, scale, dtype = ctx.cfg
        n, E = idx.shape[0], (probs.shape[1] if probs is not None else None)
        if dw is None:
            dw = torch.zeros_like(w)
        if E is None:
            E = ctx.E
        dl = torch.zeros((n, E), dtype=dtype, device=w.device) if mode == 1 else torch.empty((n, E), dtype=dtype, device=w.device)
        rc = _native.lib().pt_router_topk_bwd(None if probs is None else probs.data_ptr(), idx.data_ptr(), w.data_ptr(),
                                              dw.contiguous().float().data_ptr(),
                                              None if dprobs is None else dprobs.contiguous().data_ptr(),
                                              dl.data_ptr(), int(dtype == torch.float32), n, E, k, mode, int(renorm),
                                              float(scale), sp())
        _native.check(rc, "pt_router_topk_bwd")
        return dl, None, None, None, None


def router_topk(logits: torch.Tensor, k: int, mode: str = "softmax_topk", renorm: bool = False,
                scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    n, E = logits.shape
    if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16) and E <= 512 and k <= 16:
        m = MODES[mode]
        if m == 1:
            res = _RouterTopkSoftmax.apply(logits, k, renorm, scale)
            return res[0], res[1], None
        w, idx, probs = _RouterFn.apply(logits, k, m, renorm, scale)
        return w, idx, probs
    return router_topk_ref(logits, k, mode, renorm, scale)


class _RouterTopkSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, renorm, scale):
        n, E = logits.shape
        lg = logits.contiguous()
        idx = torch.empty((n, k), dtype=torch.int32, device=lg.device)
        w = torch.empty((n, k), dtype=torch.float32, device=lg.device)
        rc = _native.lib().pt_router_topk_fwd(lg.data_ptr(), int(lg.dtype == torch.float32), None, idx.data_ptr(),
                                              w.data_ptr(), n, E, k, 1, 0, float(scale), sp())
        _native.check(rc, "pt_router_topk_fwd")
        ctx.save_for_backward(idx, w)
        ctx.cfg = (k, scale, lg.dtype, E)
        ctx.mark_non_differentiable(idx)
        return w, idx

    @staticmethod
    def backward(ctx, dw, didx=None):
        idx, w = ctx.saved_tensors
        k, scale, dtype, E = ctx.cfg
        n = idx.shape[0]
        dl = torch.empty((n, E), dtype=dtype, device=w.device)
        rc = _native.lib().pt_router_topk_bwd(None, idx.data_ptr(), w.data_ptr(), dw.contiguous().float().data_ptr(), None,
                                              dl.data_ptr(), int(dtype == torch.float32), n, E, k, 1, 0, float(scale), sp())
        _native.check(rc, "pt_router_topk_bwd")
        return dl, None, None, None
