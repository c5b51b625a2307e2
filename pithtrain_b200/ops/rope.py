"""Rotary embeddings and the fused per-head QK-RMSNorm + RoPE on the packed QKV projection.

``qk_norm_rope(qkv, q_w, k_w, cos, sin, ...)`` takes the output of the fused q/k/v GEMM
``[tokens, (Hq + 2*Hkv) * D]`` and returns ``q[tokens,Hq,D]``, ``k[tokens,Hkv,D]`` (normalised when
weights are given, rotated by rotate-half RoPE) and ``v`` as a strided view of the input — one
kernel instead of the norm / mul / cat / rotate chain of pithtrain/models/qwen3_moe.py:140-168.
``cos``/``sin`` are ``[max_pos, D]`` tables (bf16 in the reference); ``positions`` optionally gives
each token's position (packed sequences, zigzag context parallelism).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from .common import accumulate_colsum, sp, use_native


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope_ref(x, cos, sin):
    """x [..., tokens, heads, D]; cos/sin [tokens, D]."""
    return x * cos.unsqueeze(-2) + rotate_half(x) * sin.unsqueeze(-2)


def _head_norm_ref(x, w, eps, zero_centered):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    scale = (1.0 + w.float()) if zero_centered else w.float()
    return (y * scale).to(x.dtype)


def qk_norm_rope_ref(qkv, q_w, k_w, cos, sin, Hq, Hkv, D, eps, positions=None, S=None, zero_centered=False):
    n = qkv.shape[0]
    q = qkv[:, : Hq * D].reshape(n, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(n, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].reshape(n, Hkv, D)
    if q_w is not None:
        q = _head_norm_ref(q, q_w, eps, zero_centered)
        k = _head_norm_ref(k, k_w, eps, zero_centered)
    if positions is None:
        positions = torch.arange(n, device=qkv.device) % S
    c, s = cos[positions.long()].to(q.dtype), sin[positions.long()].to(q.dtype)
    return apply_rope_ref(q, c, s), apply_rope_ref(k, c, s), v


class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, q_w, k_w, cos, sin, positions, Hq, Hkv, D, eps, S, zero_centered):
        n = qkv.shape[0]
        dev = qkv.device
        q = torch.empty((n, Hq, D), dtype=qkv.dtype, device=dev)
        k = torch.empty((n, Hkv, D), dtype=qkv.dtype, device=dev)
        has_norm = q_w is not None
        rq = torch.empty((n, Hq), dtype=torch.float32, device=dev) if has_norm else None
        rk = torch.empty((n, Hkv), dtype=torch.float32, device=dev) if has_norm else None
        pos = None if positions is None else positions.int().contiguous()
        rc = _native.lib().pt_qk_norm_rope_fwd(
            qkv.data_ptr(), q.data_ptr(), k.data_ptr(), None if not has_norm else q_w.data_ptr(),
            None if not has_norm else k_w.data_ptr(), cos.data_ptr(), sin.data_ptr(),
            None if pos is None else pos.data_ptr(), None if rq is None else rq.data_ptr(),
            None if rk is None else rk.data_ptr(), n, S, Hq, Hkv, D, qkv.stride(0), float(eps), int(zero_centered), sp())
        _native.check(rc, "pt_qk_norm_rope_fwd")
        v = qkv[:, (Hq + Hkv) * D:].view(n, Hkv, D)
        ctx.save_for_backward(qkv, q_w, k_w, cos, sin, pos, rq, rk)
        ctx.cfg = (Hq, Hkv, D, S, zero_centered)
        ctx.qw_ref, ctx.kw_ref = q_w, k_w
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, q_w, k_w, cos, sin, pos, rq, rk = ctx.saved_tensors
        Hq, Hkv, D, S, zc = ctx.cfg
        n = qkv.shape[0]
        L = _native.lib()
        dqkv = torch.empty_like(qkv)
        has_norm = q_w is not None
        grid = L.pt_qk_norm_rope_bwd_grid()
        part = torch.empty((grid, 2 * D), dtype=torch.float32, device=qkv.device) if has_norm else None
        dq = dq.contiguous() if dq is not None else torch.zeros((n, Hq, D), dtype=qkv.dtype, device=qkv.device)
        dk = dk.contiguous() if dk is not None else torch.zeros((n, Hkv, D), dtype=qkv.dtype, device=qkv.device)
        rc = L.pt_qk_norm_rope_bwd(
            dq.data_ptr(), dk.data_ptr(), qkv.data_ptr(), dqkv.data_ptr(), None if not has_norm else q_w.data_ptr(),
            None if not has_norm else k_w.data_ptr(), cos.data_ptr(), sin.data_ptr(), None if pos is None else pos.data_ptr(),
            None if rq is None else rq.data_ptr(), None if rk is None else rk.data_ptr(),
            None if part is None else part.data_ptr(), n, S, Hq, Hkv, D, qkv.stride(0), int(zc), sp())
        _native.check(rc, "pt_qk_norm_rope_bwd")
        if dv is not None:
            dqkv[:, (Hq + Hkv) * D:].copy_(dv.reshape(n, Hkv * D))
        else:
            dqkv[:, (Hq + Hkv) * D:].zero_()
        if has_norm:
            accumulate_colsum(ctx.qw_ref, part, 0, D)
            accumulate_colsum(ctx.kw_ref, part, D, 2 * D)
        return (dqkv,) + (None,) * 11


def qk_norm_rope(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                 cos: torch.Tensor, sin: torch.Tensor, Hq: int, Hkv: int, D: int, eps: float = 1e-6,
                 positions: Optional[torch.Tensor] = None, S: Optional[int] = None, zero_centered: bool = False):
    """Returns ``(q[n,Hq,D], k[n,Hkv,D], v[n,Hkv,D])`` from packed ``qkv[n, (Hq+2Hkv)*D]``."""
    if S is None:
        S = qkv.shape[0]
    if (use_native(qkv) and D in (64, 128) and cos.dtype == torch.bfloat16 and cos.shape[-1] == D
            and qkv.stride(1) == 1 and (q_w is None or q_w.dtype == torch.bfloat16)):
        return _QKNormRopeFn.apply(qkv, q_w, k_w, cos.contiguous(), sin.contiguous(), positions, Hq, Hkv, D, eps, S, zero_centered)
    return qk_norm_rope_ref(qkv, q_w, k_w, cos, sin, Hq, Hkv, D, eps, positions, S, zero_centered)
