"""The framework's own attention kernels (``csrc/attention.cu`` forward, ``csrc/attention_bwd.cu`` backward).

tcgen05 / TMEM / TMA kernels for bf16 attention in the token-major ``[B, S, H, D]`` layout the projections write:
causal or unmasked, GQA, sliding windows, packed documents (``cu_seqlens``), learned per-head sinks, and the head
dims of the four model families (64, 128, 192/128 for MLA, 256). They take the role of the reference's
FlashAttention-4 wrapper (pithtrain/operators/flash_attn_v4.py:17-99). ``ops.attention.attention`` calls
:func:`supported` and then :func:`attention`; shapes outside the kernels' range (fp32 inputs, other head dims,
CPU tensors) use the fp32 math of ``ops.attention.attention_ref``.

Windows and documents reach the kernels as one int32 vector ``row_lo[B*Sq]``: the first key each query row may see.
A key ``kp`` is visible to the query at absolute position ``qpos`` iff ``row_lo <= kp <= qpos`` (causal) or
``row_lo <= kp < Sk`` (unmasked).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

ENABLED = True
_DIMS = {(64, 64), (128, 128), (192, 128), (256, 256)}
# head-dim pairs the backward kernel covers; the others differentiate through the fp32 math
_BWD_DIMS = {(64, 64), (128, 128)}
_ROW_LO_CACHE: dict = {}


def _token_major(t: torch.Tensor) -> bool:
    """``[B, S, H, D]`` whose (H, D) block is contiguous and whose tokens are equally spaced, so that the tensor is a
    2-D ``[B*S, H*D]`` matrix with one row pitch (a slice of a fused qkv projection output qualifies)."""
    B, S, H, D = t.shape
    sb, ss, sh, sd = t.stride()
    return sd == 1 and (H == 1 or sh == D) and (B == 1 or sb == S * ss) and ss % 8 == 0 and t.data_ptr() % 16 == 0


def supported(q, k, v, causal, window_left, sinks, cu_seqlens) -> bool:
    if not (ENABLED and q.is_cuda and q.dim() == 4):
        return False
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        return False
    if (q.shape[-1], v.shape[-1]) not in _DIMS or k.shape[-1] != q.shape[-1]:
        return False
    if k.shape[2] != v.shape[2] or q.shape[2] % k.shape[2] != 0 or k.shape[1] != v.shape[1]:
        return False
    if cu_seqlens is not None and (q.shape[0] != 1 or q.shape[1] != k.shape[1]):
        return False
    return True


def row_lower_bounds(B: int, Sq: int, q_off: int, window_left: Optional[int], cu_seqlens: Optional[torch.Tensor],
                     device) -> Optional[torch.Tensor]:
    """int32 ``[B*Sq]``: first visible key of each query row, or None when every row starts at key 0."""
    has_w = window_left is not None and window_left >= 0
    if not has_w and cu_seqlens is None:
        return None
    key = (str(device), B, Sq, q_off, window_left if has_w else None)
    lo = _ROW_LO_CACHE.get(key) if cu_seqlens is None else None
    if lo is None:
        pos = torch.arange(Sq, device=device, dtype=torch.int64)
        lo = torch.zeros(Sq, device=device, dtype=torch.int64)
        if has_w:
            lo = torch.clamp(pos + q_off - int(window_left), min=0)
        if cu_seqlens is not None:
            cs = cu_seqlens.to(device=device, dtype=torch.int64)
            seg = torch.bucketize(pos, cs[1:], right=True).clamp_(max=cs.numel() - 2)
            lo = torch.maximum(lo, cs[seg])
        lo = lo.to(torch.int32).repeat(B).contiguous()
        if cu_seqlens is None:
            if len(_ROW_LO_CACHE) > 64:
                _ROW_LO_CACHE.clear()
            _ROW_LO_CACHE[key] = lo
    return lo


def _as_token_major(t: torch.Tensor) -> torch.Tensor:
    return t if _token_major(t) else t.contiguous()


def forward(q, k, v, scale: float, causal: bool, q_off: int, row_lo: Optional[torch.Tensor],
            sinks: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Launch the forward kernel: returns ``out [B,Sq,Hq,Dv]`` bf16 and ``lse [B,Hq,Sq]`` fp32."""
    from .. import _native

    q, k, v = _as_token_major(q), _as_token_major(k), _as_token_major(v)
    B, Sq, Hq, D = q.shape
    Sk, Hkv, Dv = k.shape[1], k.shape[2], v.shape[-1]
    out = torch.empty((B, Sq, Hq, Dv), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    sk = None if sinks is None else sinks.detach().float().contiguous()
    rc = _native.lib().pt_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                   _native.ptr(row_lo), _native.ptr(sk), B, Sq, Sk, Hq, Hkv, D, Dv, q.stride(1), k.stride(1),
                                   v.stride(1), out.stride(1), float(scale), int(bool(causal)), int(q_off),
                                   _native.stream_ptr())
    _native.check(rc, "pt_attn_fwd")
    return out, lse


def backward(do, q, k, v, out, lse, scale: float, causal: bool, q_off: int, row_lo: Optional[torch.Tensor]
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Launch the backward kernels: returns ``dq, dk, dv`` (bf16) and ``delta [B,Hq,Sq]`` (fp32 row sums of dO*O,
    which the sink gradient needs)."""
    from .. import _native

    q, k, v, do, out = (_as_token_major(t) for t in (q, k, v, do, out))
    lse = lse.contiguous()  # ring attention hands in halves of a longer sequence's statistics
    B, Sq, Hq, D = q.shape
    Sk, Hkv, Dv = k.shape[1], k.shape[2], v.shape[-1]
    # fp32 accumulators (dq over key tiles; dk / dv over the heads of a GQA group), zeroed in one memset
    nq, nk = B * Sq * Hq * D, B * Sk * Hkv * D
    acc = torch.zeros(nq + 2 * nk, dtype=torch.float32, device=q.device)
    dq = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    dk = torch.empty((B, Sk, Hkv, D), dtype=k.dtype, device=q.device)
    dv = torch.empty((B, Sk, Hkv, Dv), dtype=v.dtype, device=q.device)
    # the kernel reads statistics in whole 128-row tiles: pad the flat arrays by one tile
    stats = torch.zeros(2 * (B * Hq * Sq + 128), dtype=torch.float32, device=q.device)
    delta, lse2 = stats[:B * Hq * Sq + 128], stats[B * Hq * Sq + 128:]
    rc = _native.lib().pt_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                   _native.ptr(row_lo), acc.data_ptr(), acc[nq:].data_ptr(), acc[nq + nk:].data_ptr(),
                                   dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(), lse2.data_ptr(),
                                   B, Sq, Sk, Hq, Hkv, D, q.stride(1), k.stride(1), v.stride(1), out.stride(1), do.stride(1),
                                   float(scale), int(bool(causal)), int(q_off), _native.stream_ptr())
    _native.check(rc, "pt_attn_bwd")
    return dq, dk, dv, delta[:B * Hq * Sq].view(B, Hq, Sq)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sinks, row_lo, scale, causal, q_off):
        out, lse = forward(q, k, v, scale, causal, q_off, row_lo, sinks)
        ctx.save_for_backward(q, k, v, out, lse, sinks if sinks is not None else q.new_empty(0),
                              row_lo if row_lo is not None else q.new_empty(0))
        ctx.has_sinks, ctx.has_lo = sinks is not None, row_lo is not None
        ctx.scale, ctx.causal, ctx.q_off = scale, causal, q_off
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, out, lse, sinks, row_lo = ctx.saved_tensors
        sinks = sinks if ctx.has_sinks else None
        row_lo = row_lo if ctx.has_lo else None
        if (q.shape[-1], v.shape[-1]) in _BWD_DIMS and q.shape[1] % 4 == 0:  # row statistics move in 16-byte pieces
            dq, dk, dv, delta = backward(do, q, k, v, out, lse, ctx.scale, ctx.causal, ctx.q_off, row_lo)
        else:
            dq, dk, dv, delta = _math_backward(do, q, k, v, out, lse, ctx.scale, ctx.causal, ctx.q_off, row_lo)
        d_sinks = None
        if sinks is not None:
            # d lse-normalised weight of the sink column: -exp(sink - lse) * delta, summed over batch and rows
            d_sinks = -(torch.exp(sinks.float().view(1, -1, 1) - lse) * delta).sum((0, 2)).to(sinks.dtype)
        return dq, dk, dv, d_sinks, None, None, None, None


def _math_backward(do, q, k, v, out, lse, scale, causal, q_off, row_lo):
    """fp32 tensor-op backward against the kernel's ``out`` and ``lse`` for the head dims the backward kernel does not
    cover (MLA 192/128 and 256): same formulas as the kernel, O(S^2) memory."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    dof = do.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    kp = torch.arange(Sk, device=q.device).view(1, 1, 1, Sk)
    qp = (torch.arange(Sq, device=q.device) + q_off).view(1, 1, Sq, 1)
    vis = torch.ones(1, 1, Sq, Sk, dtype=torch.bool, device=q.device)
    if causal:
        vis = vis & (kp <= qp)
    if row_lo is not None:
        vis = vis & (kp >= row_lo.view(B, 1, Sq, 1))
    lse_safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - lse_safe.unsqueeze(-1)).masked_fill(~vis, 0.0)
    delta = (dof * out.float().permute(0, 2, 1, 3)).sum(-1)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta.unsqueeze(-1)) * scale
    dq = torch.matmul(ds, kf).permute(0, 2, 1, 3)
    dk = torch.matmul(ds.transpose(-1, -2), qf).view(B, Hkv, g, Sk, D).sum(2).permute(0, 2, 1, 3)
    dv = torch.matmul(p.transpose(-1, -2), dof).view(B, Hkv, g, Sk, v.shape[-1]).sum(2).permute(0, 2, 1, 3)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), delta


def attention(q, k, v, causal, scale, window_left, sinks, cu_seqlens, return_lse=False, q_off: Optional[int] = None):
    """Attention of ``q [B,Sq,Hq,D]`` against ``k [B,Sk,Hkv,D]``, ``v [B,Sk,Hkv,Dv]`` on the own kernels (autograd-aware).
    ``q_off`` is the position of query 0 relative to key 0 (default ``Sk - Sq``: the last query sees the last key)."""
    B, Sq = q.shape[0], q.shape[1]
    Sk = k.shape[1]
    if q_off is None:
        q_off = Sk - Sq
    sc = float(scale) if scale is not None else q.shape[-1] ** -0.5
    row_lo = row_lower_bounds(B, Sq, q_off, window_left, cu_seqlens, q.device)
    out, lse = _Attention.apply(q, k, v, sinks, row_lo, sc, bool(causal), int(q_off))
    return (out, lse) if return_lse else out


def block_from_pointers(q: torch.Tensor, k_ptr: int, v_ptr: int, Sk: int, Hkv: int, scale: float
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Unmasked attention of ``q [1, Sq, Hq, D]`` against ``Sk`` keys/values stored token-major and contiguous
    (``[Sk, Hkv, D]`` bf16) at raw device addresses — which may lie in another GPU's published buffer: the kernel's
    TMA loads then fetch the block over NVLink tile by tile while it computes. Returns bf16 ``out`` and fp32 ``lse``."""
    from .. import _native

    q = _as_token_major(q)
    B, Sq, Hq, D = q.shape
    assert B == 1 and q.dtype == torch.bfloat16 and (D, D) in _DIMS
    out = torch.empty((1, Sq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((1, Hq, Sq), dtype=torch.float32, device=q.device)
    rc = _native.lib().pt_attn_fwd(q.data_ptr(), k_ptr, v_ptr, out.data_ptr(), lse.data_ptr(), None, None, 1, Sq, Sk, Hq, Hkv,
                                   D, D, q.stride(1), Hkv * D, Hkv * D, out.stride(1), float(scale), 0, 0,
                                   _native.stream_ptr())
    _native.check(rc, "pt_attn_fwd")
    return out, lse
