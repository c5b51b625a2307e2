"""FP8 training path: forward and input-gradient GEMMs in block-scaled e4m3, weight gradients in bf16.

* activations / output gradients: 1x128 row-wise scales, quantised right before the GEMM (for the
  experts the quantiser gathers the token rows into expert order in the same pass);
* weights: 128x128 tile scales in both orientations, quantised once per optimizer step and cached
  (``FP8WeightCacheControl.version`` tags the cache; it is dropped before the optimizer runs);
* weight gradients stay on the bf16 K-grouped / TN kernels, which accumulate straight into the
  gradient buffers through TMA reduce-add — re-quantising ``dy`` and ``x`` along the token
  dimension for an fp8 wgrad costs two more passes over both tensors, which the shorter
  tensor-core time does not pay back at these shapes. The reference runs all three GEMMs in fp8
  through DeepGEMM (pithtrain/operators/linear.py:44-83, pithtrain/operators/grouped_linear.py:104-236).

``enable(True)`` switches every eligible :func:`pithtrain_b200.ops.linear.linear`,
:func:`pithtrain_b200.ops.grouped_linear.grouped_linear` and :func:`pithtrain_b200.ops.moe.moe_experts` call
to this path; lm_head, routers and projections narrower than 256 stay bf16, like the reference
(pithtrain/models/qwen3_moe.py:76,289).
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..dualpipe.utils import FP8WeightCacheControl, WeightGradStore
from . import gemm as G
from .common import accumulate_grad, use_native
from .quant import gemm_fp8_nt, quant_blocks, quant_rows

_ENABLED = False
MIN_DIM = 256
_WEIGHT_CACHE: Dict[Tuple[int, tuple], tuple] = {}
FP8WeightCacheControl.caches.append(_WEIGHT_CACHE)


def enable(flag: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(flag)
    _WEIGHT_CACHE.clear()


def enabled() -> bool:
    return _ENABLED


def eligible(x: torch.Tensor, weight: torch.Tensor, flag: Optional[bool] = None) -> bool:
    """Whether a ``[.., K] x [.., N, K]`` product takes the fp8 path (``flag`` False opts a module out)."""
    if flag is False or not (_ENABLED or flag is True):
        return False
    N, K = weight.shape[-2], weight.shape[-1]
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and N >= MIN_DIM and K >= MIN_DIM
            and K % 16 == 0 and N % 16 == 0 and (use_native(x) or not x.is_cuda))


def quantized_weight(w: torch.Tensor):
    """``(q, s, qT, sT)`` of ``w [N, K]`` or ``[E, N, K]``, cached until the weights change."""
    key = (w.data_ptr(), tuple(w.shape))
    hit = _WEIGHT_CACHE.get(key)
    if hit is not None and hit[0] == FP8WeightCacheControl.version:
        return hit[1]
    with torch.no_grad():
        packed = quant_blocks(w.detach().contiguous(), transposed=True)
    _WEIGHT_CACHE[key] = (FP8WeightCacheControl.version, packed)
    return packed


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, grad_targets):
        K = x.shape[-1]
        x2 = x.reshape(-1, K).contiguous()
        q, s, _, _ = quantized_weight(w)
        xq, xs = quant_rows(x2)
        y = gemm_fp8_nt(xq, xs, q, s)
        if b is not None:
            y += b
        ctx.save_for_backward(x2, w)
        ctx.grad_targets, ctx.has_bias, ctx.in_shape = grad_targets, b is not None, x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        N = w.shape[0]
        dy2 = dy.reshape(-1, N).contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            _, _, qt, st = quantized_weight(w)
            dq, ds = quant_rows(dy2)
            dx = gemm_fp8_nt(dq, ds, qt, st).view(ctx.in_shape)
        get_wgrad, bias_param = ctx.grad_targets

        def wgrad_fn(dy2=dy2, x2=x2):
            from .linear import _wgrad_into

            _wgrad_into(dy2, x2, get_wgrad())

        if ctx.has_bias and bias_param is not None:
            accumulate_grad(bias_param, dy2.float().sum(0))
        if WeightGradStore.enabled:
            WeightGradStore.put(wgrad_fn)
        else:
            wgrad_fn()
        return dx, None, None, None


class _Fp8GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offs, grad_getter):
        q, s, _, _ = quantized_weight(w)
        E = w.shape[0]
        xq, xs = quant_rows(x.contiguous(), n_rows=offs[E:E + 1])
        y = gemm_fp8_nt(xq, xs, q, s, offs=offs)
        ctx.save_for_backward(x, w, offs)
        ctx.grad_getter = grad_getter
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, offs = ctx.saved_tensors
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            _, _, qt, st = quantized_weight(w)
            dq, ds = quant_rows(dy, n_rows=offs[w.shape[0]:w.shape[0] + 1])
            dx = gemm_fp8_nt(dq, ds, qt, st, offs=offs)
        get = ctx.grad_getter

        def wgrad_fn(dy=dy, x=x, offs=offs):
            G.grouped_gemm_tn(dy, x, offs, get(), accumulate=True)

        if WeightGradStore.enabled:
            WeightGradStore.put(wgrad_fn)
        else:
            wgrad_fn()
        return dx, None, None, None


def fp8_linear_apply(x, weight, bias, grad_targets):
    return _Fp8LinearFn.apply(x, weight, bias, grad_targets)


def fp8_grouped_linear_apply(x, weight, offs, grad_getter):
    return _Fp8GroupedLinearFn.apply(x, weight, offs, grad_getter)


def _module_classes():
    from .grouped_linear import GroupedLinear
    from .linear import Linear

    class FP8Linear(Linear):
        """``Linear`` that always takes the fp8 path (when its shape allows), whatever the global switch."""

        fp8 = True

    class FP8GroupedLinear(GroupedLinear):
        fp8 = True

    return FP8Linear, FP8GroupedLinear


FP8Linear, FP8GroupedLinear = _module_classes()
