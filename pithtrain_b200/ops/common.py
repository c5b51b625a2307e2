"""Shared helpers for operators: native-path predicate and gradient accumulation into main grads."""

from __future__ import annotations

import torch

from .. import _native


def use_native(*tensors: torch.Tensor) -> bool:
    """True when the sm_100a kernels apply: CUDA tensors in bf16. Raises if the library is absent."""
    t = tensors[0]
    if not t.is_cuda:
        return False
    if t.dtype != torch.bfloat16:
        return False
    _native.lib()  # raises NativeLibraryMissing on a GPU box without the built library
    return True


def accumulate_grad(p: torch.Tensor, g: torch.Tensor) -> None:
    """Add ``g`` to the gradient accumulator of parameter ``p``.

    Parameters managed by a flat shard group carry ``main_grad`` (a view into the group's flat
    gradient buffer, possibly fp32); plain parameters fall back to ``.grad``.
    """
    mg = getattr(p, "main_grad", None)
    if mg is not None:
        mg.add_(g.reshape(mg.shape))
    elif p.grad is None:
        p.grad = g.reshape(p.shape).to(p.dtype).clone()
    else:
        p.grad.add_(g.reshape(p.shape))


def grad_buffer(p: torch.Tensor) -> torch.Tensor:
    """Tensor that kernels may accumulate into directly (creates a zero ``.grad`` when needed)."""
    mg = getattr(p, "main_grad", None)
    if mg is not None:
        return mg
    if p.grad is None:
        p.grad = torch.zeros_like(p)
    return p.grad


def sp() -> int:
    return _native.stream_ptr()
