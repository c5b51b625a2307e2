"""Attention entry points (BSHD layout): causal GQA/MHA with optional sliding window, learned
per-head sinks, asymmetric q/v head dims (MLA) and packed sequences.

``attention(q, k, v, ...)`` returns ``out[B,S,Hq,Dv]``; ``attention_with_lse`` also returns the
log-sum-exp ``[B,Hq,S]`` that ring attention merges on. On GPUs the work is done by the tcgen05 kernels of
``csrc/attention.cu`` / ``csrc/attention_bwd.cu``. The feature set is that of the reference's
FlashAttention-4 wrapper (pithtrain/operators/flash_attn_v4.py:17-99): ``causal``,
``window=(left, 0)``, ``learnable_sink``, ``cu_seqlens``.
``attention_ref`` is the fp32 oracle.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def _mask(Sq: int, Sk: int, causal: bool, window_left: Optional[int], device, q_offset: int = 0,
          seg_q: Optional[torch.Tensor] = None, seg_k: Optional[torch.Tensor] = None) -> torch.Tensor:
    qi = torch.arange(Sq, device=device).unsqueeze(1) + q_offset
    ki = torch.arange(Sk, device=device).unsqueeze(0)
    m = torch.ones(Sq, Sk, dtype=torch.bool, device=device)
    if causal:
        m &= ki <= qi
    if window_left is not None and window_left >= 0:
        m &= ki >= qi - window_left
    if seg_q is not None:
        m &= seg_q.unsqueeze(1) == seg_k.unsqueeze(0)
    return m


def segments_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    pos = torch.arange(total, device=cu_seqlens.device)
    return torch.bucketize(pos, cu_seqlens[1:].long(), right=True)


def attention_ref(q, k, v, causal=True, scale=None, window_left=None, sinks=None, cu_seqlens=None,
                  return_lse=False, mask=None):
    """fp32 math attention. q [B,Sq,Hq,D], k [B,Sk,Hkv,D], v [B,Sk,Hkv,Dv]."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else D ** -0.5
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)  # B,Hq,Sq,D
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if mask is None:
        seg = None
        if cu_seqlens is not None:
            seg = segments_from_cu_seqlens(cu_seqlens, Sq)
        mask = _mask(Sq, Sk, causal, window_left, q.device, q_offset=Sk - Sq, seg_q=seg, seg_k=seg)
    s = s.masked_fill(~mask, float("-inf"))
    if sinks is not None:
        sk = sinks.float().view(1, Hq, 1, 1).expand(B, Hq, Sq, 1)
        s_all = torch.cat([s, sk], dim=-1)
        lse = torch.logsumexp(s_all, dim=-1)
    else:
        lse = torch.logsumexp(s, dim=-1)
    lse_safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - lse_safe.unsqueeze(-1))
    out = torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)
    if return_lse:
        return out, lse
    return out


def attention_window_blocked(q, k, v, window_left: int, scale=None, sinks=None, seg: Optional[torch.Tensor] = None,
                             block: int = 128) -> torch.Tensor:
    """Causal sliding-window attention in ``O(S * (window + block))`` instead of ``O(S^2)``.

    Queries are cut into blocks of ``block``; block ``i`` only sees the keys of the ``ceil(window/block)`` previous
    blocks and its own, so scores are ``[B, H, S/block, block, span]`` with ``span = (ceil(window/block)+1)*block``
    (GPT-OSS: window 127/128 -> span 256). Plain tensor ops with autograd; same math as :func:`attention_ref`
    (fp32 scores, optional per-head sinks in the softmax denominator, optional document ids ``seg[S]``).
    """
    B, S, Hq, D = q.shape
    Hkv, Dv = k.shape[2], v.shape[-1]
    g = Hq // Hkv
    scale = scale if scale is not None else D ** -0.5
    nb = S // block
    back = (window_left + block - 1) // block  # previous blocks a query block can reach
    span = (back + 1) * block
    qf = q.float().view(B, nb, block, Hkv, g, D).permute(0, 3, 4, 1, 2, 5)  # B,Hkv,g,nb,block,D
    pad = back * block

    def windows(t: torch.Tensor) -> torch.Tensor:  # [B,S,Hkv,d] -> [B,Hkv,nb,span,d]
        tp = F.pad(t.float().permute(0, 2, 1, 3), (0, 0, pad, 0))  # B,Hkv,pad+S,d
        return tp.unfold(2, span, block).permute(0, 1, 2, 4, 3)  # windows start at block i - back

    kw, vw = windows(k), windows(v)
    s = torch.einsum("bhgnqd,bhnkd->bhgnqk", qf, kw) * scale  # B,Hkv,g,nb,block,span
    dev = q.device
    qpos = (torch.arange(nb, device=dev) * block).view(nb, 1, 1) + torch.arange(block, device=dev).view(1, block, 1)
    kpos = (torch.arange(nb, device=dev) * block - pad).view(nb, 1, 1) + torch.arange(span, device=dev).view(1, 1, span)
    m = (kpos <= qpos) & (kpos >= qpos - window_left) & (kpos >= 0)
    if seg is not None:
        segp = F.pad(seg, (pad, 0), value=-1)
        kseg = segp.unfold(0, span, block)  # nb, span
        qseg = seg.view(nb, block)
        m = m & (kseg.unsqueeze(1) == qseg.unsqueeze(2))
    s = s.masked_fill(~m, float("-inf"))
    if sinks is not None:
        sk = sinks.float().view(1, Hkv, g, 1, 1, 1).expand(B, Hkv, g, nb, block, 1)
        lse = torch.logsumexp(torch.cat([s, sk], dim=-1), dim=-1, keepdim=True)
    else:
        lse = torch.logsumexp(s, dim=-1, keepdim=True)
    lse = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - lse)
    out = torch.einsum("bhgnqk,bhnkd->bhgnqd", p, vw)  # B,Hkv,g,nb,block,Dv
    return out.permute(0, 3, 4, 1, 2, 5).reshape(B, S, Hq, Dv).to(q.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              scale: Optional[float] = None, window_left: Optional[int] = None,
              sinks: Optional[torch.Tensor] = None, cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 tensors on a GPU run on the framework's own tcgen05 kernels (``ops/attention_native.py``: every mask and
    head dim the model families use); everything else (CPU, fp32, other head dims) on the fp32 math, in the blocked
    O(S * window) form for long sliding-window sequences."""
    from . import attention_native

    if attention_native.supported(q, k, v, causal, window_left, sinks, cu_seqlens):
        return attention_native.attention(q, k, v, causal, scale, window_left, sinks, cu_seqlens)
    S = q.shape[1]
    if causal and window_left is not None and window_left >= 0 and S == k.shape[1] and S % 128 == 0 and S > 2 * (window_left + 128):
        seg = segments_from_cu_seqlens(cu_seqlens, S) if cu_seqlens is not None else None
        return attention_window_blocked(q, k, v, window_left, scale, sinks, seg)
    return attention_ref(q, k, v, causal, scale, window_left, sinks, cu_seqlens)


def attention_with_lse(q, k, v, causal=True, scale=None, window_left=None, sinks=None, mask=None
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of a q block against a kv block returning (out, lse[B,Hq,Sq]); used by the ring."""
    from . import attention_native

    if mask is None and attention_native.supported(q, k, v, causal, window_left, sinks, None):
        return attention_native.attention(q, k, v, causal, scale, window_left, sinks, None, return_lse=True)
    return attention_ref(q, k, v, causal, scale, window_left, sinks, None, return_lse=True, mask=mask)


def flash_attn_func(q, k, v, softmax_scale=None, causal=True, window_size=(None, None), learnable_sink=None):
    """Signature-compatible alias of the reference's ``flash_attn_func``."""
    wl = window_size[0] if window_size and window_size[0] is not None and window_size[0] >= 0 else None
    return attention(q, k, v, causal=causal, scale=softmax_scale, window_left=wl, sinks=learnable_sink)


def flash_attn_varlen_func(q, k, v, cu_seqlens, softmax_scale=None, causal=True, window_size=(None, None),
                           learnable_sink=None):
    """Packed-sequence form: q/k/v are ``[total, H, D]`` and ``cu_seqlens`` marks document starts."""
    wl = window_size[0] if window_size and window_size[0] is not None and window_size[0] >= 0 else None
    out = attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), causal=causal, scale=softmax_scale,
                    window_left=wl, sinks=learnable_sink, cu_seqlens=cu_seqlens)
    return out.squeeze(0)
