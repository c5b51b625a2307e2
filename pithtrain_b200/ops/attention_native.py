"""Hand-written sm_100a attention kernels (tcgen05 + TMEM); selected when the shape is supported."""

from __future__ import annotations

import torch

from .. import _native

ENABLED = True


def supported(q, k, v, causal, window_left, sinks, cu_seqlens) -> bool:
    if not ENABLED or not q.is_cuda:
        return False
    L = _native.lib()
    if not hasattr(L, "pt_attn_fwd"):
        return False
    from .attention_kernels import shape_supported

    return shape_supported(q, k, v, causal, window_left, sinks, cu_seqlens)


def attention(q, k, v, causal, scale, window_left, sinks, cu_seqlens, return_lse=False):
    from .attention_kernels import attention_fn

    return attention_fn(q, k, v, causal, scale, window_left, sinks, cu_seqlens, return_lse)
