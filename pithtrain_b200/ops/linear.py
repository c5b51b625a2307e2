"""Dense linear layers on the tcgen05 GEMMs with deferred weight gradients.

``linear(x, w, b)`` runs forward ``x @ w.T`` (gemm_nt), dgrad ``dy @ w`` (gemm_nn) and wgrad
``dy.T @ x`` (gemm_tn). The wgrad GEMM accumulates straight into the parameter's gradient buffer
(epilogue ``D += acc``) and, while ``WeightGradStore.enabled``, is queued as a closure so the
pipeline can run it in a zero-bubble W phase. Parameters that sit next to each other in one flat
buffer can be multiplied as a single fused weight (q/k/v): see :class:`FusedWeights`.
Reference counterpart: the ``training.Linear`` binding (pithtrain/modules/training.py:383-385) and
pithtrain/operators/linear.py:170-208.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn

from ..dualpipe.utils import WeightGradStore
from . import gemm as G
from .common import accumulate_grad, grad_buffer, use_native


def _wgrad_into(dy2: torch.Tensor, x2: torch.Tensor, target: torch.Tensor) -> None:
    """target[N,K] += dy2[M,N].T @ x2[M,K]."""
    if use_native(dy2) and x2.dtype == torch.bfloat16 and target.is_contiguous() and dy2.shape[1] % 8 == 0 \
            and x2.shape[1] % 8 == 0 and dy2.shape[0] % 8 == 0:
        G.gemm_tn(dy2, x2, out=target, accumulate=True)
    else:
        target.add_((dy2.float().t() @ x2.float()).to(target.dtype))


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, grad_targets):
        """``grad_targets`` = (weight_grad_buffer_getter, bias_param) resolved lazily at backward."""
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if use_native(x2) and w.dtype == torch.bfloat16 and K % 8 == 0 and w.shape[0] % 8 == 0:
            x2 = x2.contiguous()
            y = G.gemm_nt(x2, w)
            if b is not None:
                y += b
        else:
            y = torch.nn.functional.linear(x2, w, b)
        ctx.save_for_backward(x2, w)
        ctx.grad_targets = grad_targets
        ctx.has_bias = b is not None
        ctx.in_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        N = w.shape[0]
        dy2 = dy.reshape(-1, N)
        if use_native(dy2) and w.dtype == torch.bfloat16 and N % 8 == 0 and w.shape[1] % 8 == 0:
            dy2 = dy2.contiguous()
            dx = G.gemm_nn(dy2, w) if ctx.needs_input_grad[0] else None
        else:
            dx = (dy2 @ w) if ctx.needs_input_grad[0] else None
        get_wgrad, bias_param = ctx.grad_targets

        def wgrad_fn(dy2=dy2, x2=x2):
            _wgrad_into(dy2, x2, get_wgrad())

        if ctx.has_bias and bias_param is not None:
            accumulate_grad(bias_param, dy2.float().sum(0))
        if WeightGradStore.enabled:
            WeightGradStore.put(wgrad_fn)
        else:
            wgrad_fn()
        return (dx.view(ctx.in_shape) if dx is not None else None), None, None, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           weight_param: Optional[torch.Tensor] = None, grad_getter=None, fp8: Optional[bool] = None) -> torch.Tensor:
    """``x @ weight.T + bias`` with manual weight-gradient accumulation.

    ``weight`` may be a plain view covering several parameters; then ``grad_getter`` returns the
    matching view of their gradient buffers.
    """
    wp = weight if weight_param is None else weight_param
    if grad_getter is None:
        grad_getter = lambda: grad_buffer(wp)  # noqa: E731
    if not x.requires_grad and torch.is_grad_enabled():
        # the weight gradient is produced inside backward(), which autograd only calls when some
        # input requires grad
        x = x.detach().requires_grad_()
    from . import fp8_linear

    if fp8_linear.eligible(x, weight, fp8):
        return fp8_linear.fp8_linear_apply(x, weight, bias, (grad_getter, bias))
    return _LinearFn.apply(x, weight, bias, (grad_getter, bias))


class Linear(nn.Linear):
    """``nn.Linear`` whose matmuls run on the sm_100a GEMM and whose wgrad can be deferred."""

    fp8: Optional[bool] = None  # None: follow the global fp8 switch; False: always bf16; True: always fp8

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, self.bias, fp8=self.fp8)


class FusedWeights:
    """Several parameters stored inside one tensor so a single GEMM can use them all.

    Two layouts: ``"rows"`` — ``[out_i, in]`` matrices stacked along dim 0 (q/k/v, dense gate/up);
    ``"pair"`` — two ``[E, I, H]`` expert stacks interleaved as ``[E, 2, I, H]`` so each expert's
    gate and up rows are adjacent (the fused ``[E, 2I, H]`` operand of the grouped GEMM).

    ``bind()`` allocates the fused tensor and re-points each parameter's ``data`` at its view. A
    flat shard group later re-binds the same parameters into its own buffers through
    :meth:`rebind`. ``weight()`` returns the fused view, or ``None`` if the views are no longer in
    place (e.g. after ``module.to()``); ``ensure()`` re-fuses in that case.
    """

    def __init__(self, params: Sequence[nn.Parameter], layout: str = "rows"):
        self.params: List[nn.Parameter] = list(params)
        self.layout = layout
        self.fused: Optional[torch.Tensor] = None
        self.fused_grad: Optional[torch.Tensor] = None
        self.bind()

    # -- geometry
    def fused_shape(self) -> tuple:
        p0 = self.params[0]
        if self.layout == "rows":
            return (sum(p.shape[0] for p in self.params),) + tuple(p0.shape[1:])
        assert len(self.params) == 2 and self.params[0].shape == self.params[1].shape
        E, I, H = p0.shape
        return (E, 2, I, H)

    def views(self, fused: torch.Tensor) -> List[torch.Tensor]:
        if self.layout == "rows":
            out, off = [], 0
            for p in self.params:
                out.append(fused[off:off + p.shape[0]])
                off += p.shape[0]
            return out
        return [fused[:, 0], fused[:, 1]]

    def gemm_view(self, fused: torch.Tensor) -> torch.Tensor:
        if self.layout == "rows":
            return fused
        E, _, I, H = fused.shape
        return fused.view(E, 2 * I, H)

    @property
    def numel(self) -> int:
        return sum(p.numel() for p in self.params)

    # -- binding
    def bind(self) -> None:
        p0 = self.params[0]
        fused = torch.empty(self.fused_shape(), dtype=p0.dtype, device=p0.device)
        self.rebind(fused, None)

    def rebind(self, fused: torch.Tensor, fused_grad: Optional[torch.Tensor], copy: bool = True,
               swap=None) -> None:
        """Point the parameters at views of ``fused`` (and their ``main_grad`` at ``fused_grad``).

        Parameters built on the meta device cannot adopt real storage; they are replaced by new
        ``nn.Parameter`` objects and ``swap(old, new)`` is called so the owner module can re-register.
        """
        fused = fused.view(self.fused_shape())
        gviews = [None] * len(self.params)
        if fused_grad is not None:
            fused_grad = fused_grad.view(self.fused_shape())
            gviews = self.views(fused_grad)
        with torch.no_grad():
            for i, (p, view) in enumerate(zip(self.params, self.views(fused))):
                if p.is_meta and not view.is_meta:
                    q = nn.Parameter(view, requires_grad=p.requires_grad)
                    for attr in ("_init_fill", "_init_fn"):
                        if hasattr(p, attr):
                            setattr(q, attr, getattr(p, attr))
                    if swap is not None:
                        swap(p, q)
                    self.params[i] = p = q
                else:
                    if copy and not p.is_meta:
                        view.copy_(p.data)
                    p.data = view
                if gviews[i] is not None:
                    p.main_grad = gviews[i]
                p._fusion = (self, i)
        self.fused, self.fused_grad = fused, fused_grad

    def _in_place(self, tensors, fused) -> bool:
        if fused is None:
            return False
        for t, view in zip(tensors, self.views(fused)):
            if t is None or t.data_ptr() != view.data_ptr() or t.stride() != view.stride() or t.dtype != view.dtype:
                return False
        return True

    def weight(self) -> Optional[torch.Tensor]:
        if not self._in_place([p.data for p in self.params], self.fused):
            return None
        return self.gemm_view(self.fused)

    def ensure(self) -> torch.Tensor:
        """Fused GEMM operand, re-fusing first if the parameters were moved."""
        w = self.weight()
        if w is None:
            self.fused_grad = None
            self.bind()
            w = self.gemm_view(self.fused)
        return w

    def grad(self) -> torch.Tensor:
        """Fused gradient buffer (main grads when managed by a shard group, else fused ``.grad``)."""
        if self.fused_grad is not None and getattr(self.params[0], "main_grad", None) is not None:
            return self.gemm_view(self.fused_grad)
        if not self._in_place([p.grad for p in self.params], self.fused_grad):
            g = torch.zeros(self.fused_shape(), dtype=self.fused.dtype, device=self.fused.device)
            for p, gview in zip(self.params, self.views(g)):
                if p.grad is not None:
                    gview.copy_(p.grad)
                p.grad = gview
            self.fused_grad = g
        return self.gemm_view(self.fused_grad)


def fused_linear(x: torch.Tensor, fw: FusedWeights, biases: Sequence[Optional[torch.Tensor]] | None = None):
    """One GEMM against all weights of ``fw`` when they are adjacent, else one GEMM per weight."""
    w = fw.ensure()
    bias = None
    if biases is not None and any(b is not None for b in biases):
        bias = _CatBias.apply(*biases)
    y = linear(x, w, None, weight_param=None, grad_getter=fw.grad)
    if bias is not None:
        y = y + bias
    return y


class _CatBias(torch.autograd.Function):
    """cat of bias parameters whose backward accumulates into their gradient buffers."""

    @staticmethod
    def forward(ctx, *biases):
        ctx.biases = biases
        return torch.cat([b.detach() for b in biases])

    @staticmethod
    def backward(ctx, g):
        off = 0
        for b in ctx.biases:
            accumulate_grad(b, g[off:off + b.numel()])
            off += b.numel()
        return tuple(None for _ in ctx.biases)


def __getattr__(name: str):
    # ``FP8Linear`` lives with the fp8 path; the reference exports it from this module
    # (pithtrain/operators/linear.py:170), so it resolves here too, lazily to keep the imports acyclic.
    if name == "FP8Linear":
        from .fp8_linear import FP8Linear

        return FP8Linear
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
