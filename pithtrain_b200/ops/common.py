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


def accumulate_colsum(p: torch.Tensor, part: torch.Tensor, lo: int = 0, hi: int | None = None) -> None:
    """``grad(p) += part[:, lo:hi].sum(0)`` for fp32 per-block partial sums ``part [G, C]``.

    On CUDA with a flat gradient buffer this is one kernel that sums the partials and accumulates in
    place; otherwise the reduction and :func:`accumulate_grad`.
    """
    hi = part.shape[1] if hi is None else hi
    mg = getattr(p, "main_grad", None)
    if (mg is not None and mg.is_cuda and part.is_cuda and mg.is_contiguous() and part.stride(1) == 1
            and part.dtype == torch.float32 and mg.dtype in (torch.float32, torch.bfloat16) and mg.numel() == hi - lo):
        rc = _native.lib().pt_colsum_accumulate(part.data_ptr() + 4 * lo, part.shape[0], part.stride(0), hi - lo,
                                                mg.data_ptr(), int(mg.dtype == torch.float32), _native.stream_ptr())
        _native.check(rc, "pt_colsum_accumulate")
        return
    accumulate_grad(p, part[:, lo:hi].sum(0))
