"""Attention entry points with the signatures of the reference's FlashAttention-4 wrapper
(pithtrain/operators/flash_attn_v4.py:54,97): ``softmax_scale`` is positional and the packed form takes ``max_seqlen``."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import attention as _A

__all__ = ["flash_attn_func", "flash_attn_varlen_func"]


def flash_attn_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float, causal: bool = False,
                    window_size: Tuple[Optional[int], Optional[int]] = (None, None),
                    learnable_sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _A.flash_attn_func(q, k, v, softmax_scale=softmax_scale, causal=causal, window_size=window_size,
                              learnable_sink=learnable_sink)


def flash_attn_varlen_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                           softmax_scale: float, causal: bool = False,
                           window_size: Tuple[Optional[int], Optional[int]] = (None, None),
                           learnable_sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    del max_seqlen  # nothing here is sized by it
    return _A.flash_attn_varlen_func(q, k, v, cu_seqlens, softmax_scale=softmax_scale, causal=causal,
                                     window_size=window_size, learnable_sink=learnable_sink)
