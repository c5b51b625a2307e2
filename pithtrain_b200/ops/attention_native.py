"""Plug-in point for an attention kernel of this framework's own.

``ops.attention.attention`` asks :func:`supported` first and falls back to the library kernel (cuDNN SDPA) and
then to the fp32 math when no implementation is registered or the shape is outside its range. An implementation
registers a predicate and a function with the signatures below; none ships at present, so this module only keeps
the dispatch contract in one place.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

ENABLED = True
_IMPL: Optional[Tuple[Callable[..., bool], Callable]] = None


def register(shape_supported: Callable[..., bool], attention_fn: Callable) -> None:
    """``shape_supported(q, k, v, causal, window_left, sinks, cu_seqlens) -> bool`` and
    ``attention_fn(q, k, v, causal, scale, window_left, sinks, cu_seqlens, return_lse) -> out | (out, lse)``."""
    global _IMPL
    _IMPL = (shape_supported, attention_fn)


def supported(q, k, v, causal, window_left, sinks, cu_seqlens) -> bool:
    return bool(ENABLED and _IMPL is not None and q.is_cuda and _IMPL[0](q, k, v, causal, window_left, sinks, cu_seqlens))


def attention(q, k, v, causal, scale, window_left, sinks, cu_seqlens, return_lse=False):
    assert _IMPL is not None
    return _IMPL[1](q, k, v, causal, scale, window_left, sinks, cu_seqlens, return_lse)
