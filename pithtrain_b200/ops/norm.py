"""RMSNorm with an optional fused residual add, forward and backward.

``rmsnorm(x, w, eps)`` returns ``norm(x) * w``; with ``residual`` it returns ``(norm(h) * w, h)``
where ``h = x + residual`` — the pre-norm residual pattern of every decoder layer — in one pass
over memory. ``zero_centered`` uses ``(1 + w)`` as the scale (Qwen3.5,
pithtrain/models/qwen35_moe.py:24-34). The weight gradient is accumulated into the parameter's
gradient buffer directly.
"""

from __future__ import annotations

import torch

from .. import _native
from .common import accumulate_colsum, accumulate_grad, sp, use_native


def rmsnorm_ref(x, w, eps, residual=None, zero_centered=False):
    h = x if residual is None else x + residual
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    scale = (1.0 + w.float()) if zero_centered else w.float()
    y = (hf * rstd * scale).to(x.dtype)
    return (y, h) if residual is not None else y


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual, zero_centered):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        n = x2.shape[0]
        ctx.has_res = residual is not None
        ctx.zero_centered = zero_centered
        ctx.shape = shape
        if use_native(x2) and H % 8 == 0 and H <= 8192 and w.dtype == torch.bfloat16:
            x2 = x2.contiguous()
            r2 = residual.reshape(-1, H).contiguous() if residual is not None else None
            y = torch.empty_like(x2)
            h = torch.empty_like(x2) if r2 is not None else x2
            rstd = torch.empty(n, dtype=torch.float32, device=x.device)
            rc = _native.lib().pt_rmsnorm_fwd(x2.data_ptr(), None if r2 is None else r2.data_ptr(), w.data_ptr(),
                                               y.data_ptr(), None if r2 is None else h.data_ptr(), rstd.data_ptr(),
                                               n, H, float(eps), int(zero_centered), sp())
            _native.check(rc, "pt_rmsnorm_fwd")
            ctx.native = True
        else:
            h = x2 if residual is None else x2 + residual.reshape(-1, H)
            hf = h.float()
            rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
            scale = (1.0 + w.float()) if zero_centered else w.float()
            y = (hf * rstd[:, None] * scale).to(x.dtype)
            ctx.native = False
        ctx.save_for_backward(h, w, rstd)
        ctx.w_ref = w
        if residual is not None:
            return y.view(shape), h.view(shape)
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        h, w, rstd = ctx.saved_tensors
        H = h.shape[-1]
        n = h.shape[0]
        dy2 = dy.reshape(-1, H)
        dh2 = dh.reshape(-1, H) if (ctx.has_res and dh is not None) else None
        if ctx.native:
            dy2 = dy2.contiguous()
            dh2 = dh2.contiguous() if dh2 is not None else None
            L = _native.lib()
            grid = L.pt_rmsnorm_bwd_grid(n)
            dx = torch.empty_like(h)
            part = torch.empty((grid, H), dtype=torch.float32, device=h.device)
            rc = L.pt_rmsnorm_bwd(dy2.data_ptr(), None if dh2 is None else dh2.data_ptr(), h.data_ptr(), w.data_ptr(),
                                  rstd.data_ptr(), dx.data_ptr(), part.data_ptr(), n, H, int(ctx.zero_centered), sp())
            _native.check(rc, "pt_rmsnorm_bwd")
            dw = None
            if ctx.needs_input_grad[1]:
                accumulate_colsum(ctx.w_ref, part)
        else:
            hf, g = h.float(), dy2.float()
            xh = hf * rstd[:, None]
            scale = (1.0 + w.float()) if ctx.zero_centered else w.float()
            dw = (g * xh).sum(0)
            gw = g * scale
            dx = rstd[:, None] * (gw - xh * (gw * xh).mean(-1, keepdim=True))
            if dh2 is not None:
                dx = dx + dh2.float()
            dx = dx.to(h.dtype)
        if ctx.needs_input_grad[1] and dw is not None:
            accumulate_grad(ctx.w_ref, dw)
        dx = dx.view(ctx.shape)
        return dx, None, None, (dx if ctx.has_res else None), None


def rmsnorm(x, w, eps=1e-6, residual=None, zero_centered=False):
    return _RMSNormFn.apply(x, w, eps, residual, zero_centered)


class RMSNorm(torch.nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, zero_centered: bool = False, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.zero_centered = zero_centered
        init = torch.zeros if zero_centered else torch.ones
        self.weight = torch.nn.Parameter(init(dim, device=device, dtype=dtype))
        self.weight._init_fill = 0.0 if zero_centered else 1.0

    def forward(self, x, residual=None):
        return rmsnorm(x, self.weight, self.eps, residual, self.zero_centered)
