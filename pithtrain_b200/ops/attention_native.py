"""Plug-in point for an attention kernel of this framework's own.

``ops.attention.attention`` asks :func:`supported` first and falls back to the library kernel (cuDNN SDPA) and
then to the fp32 math when no implementation is registered or the shape is outside its range. An implementation
registers a predicate and a function with the signatures below.

The one implementation in the tree is the causal GQA forward of ``csrc/attention.cu`` (head dim 128, tcgen05 / TMEM,
one softmax thread per row) with the library flash backward against the kernel's ``out`` and log-sum-exp. The
kernel compiles but has not been validated on hardware yet, so it is registered only when
``PITHTRAIN_OWN_ATTENTION=1`` is set; without the switch this module changes nothing. ``PITHTRAIN_OWN_ATTENTION=ring``
also lets ring attention hand the kernel the address of a peer's published K/V block (:func:`block_from_pointers`),
so that the block is fetched by the kernel's own TMA loads while it is being consumed.
"""

from __future__ import annotations

import os
from typing import Callable, Optional, Tuple

import torch

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


# ------------------------------------------------------------------------------------------------
# causal GQA forward of csrc/attention.cu
# ------------------------------------------------------------------------------------------------
def causal_d128_supported(q, k, v, causal, window_left, sinks, cu_seqlens) -> bool:
    """Self-attention over whole sequences: causal, no window, no sinks, one document per row, head dim 128 for
    q, k and v, sequence a multiple of 128, bf16, token-major tensors whose rows start on 16-byte boundaries."""
    if not causal or window_left is not None or sinks is not None or cu_seqlens is not None:
        return False
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        return False
    B, S, Hq, D = q.shape
    if D != 128 or k.shape[-1] != 128 or v.shape[-1] != 128 or k.shape[1] != S or S % 128 != 0:
        return False
    if k.shape[2] != v.shape[2] or Hq % k.shape[2] != 0:
        return False
    return all(_token_major(t) for t in (q, k, v))


def _token_major(t: torch.Tensor) -> bool:
    """``[B, S, H, D]`` whose (H, D) block is contiguous and whose tokens are equally spaced, so that the tensor is a
    2-D ``[B*S, H*D]`` matrix with one row pitch (a slice of a fused qkv projection output qualifies)."""
    B, S, H, D = t.shape
    sb, ss, sh, sd = t.stride()
    return sd == 1 and sh == D and (B == 1 or sb == S * ss) and ss % 8 == 0 and t.data_ptr() % 16 == 0


class _CausalD128(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        from .. import _native

        B, S, Hq, D = q.shape
        Hkv = k.shape[2]
        out = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
        rc = _native.lib().pt_attn_fwd_causal(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S,
                                              Hq, Hkv, q.stride(1), k.stride(1), v.stride(1), out.stride(1), float(scale),
                                              _native.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"pt_attn_fwd_causal failed with code {rc}")
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale = scale
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        from .ring_attention import _lib_block_bwd

        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = _lib_block_bwd(do, q, k, v, out, lse, ctx.scale, True)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None


def causal_d128_attention(q, k, v, causal, scale, window_left, sinks, cu_seqlens, return_lse=False):
    sc = scale if scale is not None else q.shape[-1] ** -0.5
    out, lse = _CausalD128.apply(q, k, v, sc)
    return (out, lse) if return_lse else out


def block_from_pointers(q: torch.Tensor, k_ptr: int, v_ptr: int, Sk: int, Hkv: int, scale: float
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Unmasked attention of ``q [1, Sq, Hq, 128]`` against ``Sk`` keys/values stored token-major and contiguous
    (``[Sk, Hkv, 128]`` bf16) at raw device addresses — which may lie in another GPU's published buffer: the kernel's
    TMA loads then fetch the block over NVLink tile by tile while it computes. Returns fp32 ``out`` and ``lse``."""
    from .. import _native

    B, Sq, Hq, D = q.shape
    assert B == 1 and D == 128 and q.dtype == torch.bfloat16 and Sq % 128 == 0 and Sk % 128 == 0 and _token_major(q)
    out = torch.empty((1, Sq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((1, Hq, Sq), dtype=torch.float32, device=q.device)
    rc = _native.lib().pt_attn_fwd_block(q.data_ptr(), k_ptr, v_ptr, out.data_ptr(), lse.data_ptr(), 1, Sq, Sk, Hq, Hkv,
                                         q.stride(1), Hkv * D, Hkv * D, out.stride(1), float(scale), _native.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"pt_attn_fwd_block failed with code {rc}")
    return out.float(), lse


MODE = os.environ.get("PITHTRAIN_OWN_ATTENTION", "0")
# "1": causal self-attention on the own kernel; "ring": additionally, context-parallel steps read the peer's published
# K/V in place through the block form of the kernel (ops/ring_attention.py) instead of copying the block first.
RING_DIRECT = MODE == "ring"
if MODE in ("1", "ring"):
    register(causal_d128_supported, causal_d128_attention)
