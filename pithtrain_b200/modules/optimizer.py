"""Muon and AdamW over owner-sharded parameters.

Muon: fp32 SGD momentum, Nesterov blend, quintic Newton-Schulz orthogonalisation (5 steps, bf16,
batched over stacked experts), Moonlight scale ``0.2*sqrt(max(n,m))``, decoupled weight decay —
the update rule of pithtrain/modules/optimizer.py:34-63,155-211. Because a parameter's owner holds
the whole matrix and its fully reduced gradient (see :mod:`pithtrain_b200.parallel.flat_shard`),
Newton-Schulz runs locally on ~1/G of the weights per rank and the regular parameter all-gather
publishes the result; the reference's gather-per-weight and owner broadcasts have no counterpart.

Both optimizers read ``p.main_grad`` when present (flat accumulators, possibly fp32 for bf16
parameters) and ``p.grad`` otherwise, and skip parameters this rank does not own.
"""

from __future__ import annotations

from typing import Iterable, List, Optional

import torch

from ..ops import gemm as G


def _grad_of(p: torch.Tensor) -> Optional[torch.Tensor]:
    g = getattr(p, "main_grad", None)
    return g if g is not None else p.grad


def _owned(p: torch.Tensor) -> bool:
    grp = getattr(p, "_shard_group", None)
    return True if grp is None else grp.is_owned(p)


def zeropower_via_newtonschulz5(Gm: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz iteration towards the orthogonal polar factor, batched over leading dims.

    Works on the wide orientation, pre-scales by the Frobenius norm so the spectral norm is <= 1, and
    iterates ``X <- aX + (bA + cA^2)X`` with ``A = X X^T`` in bf16.
    """
    assert Gm.ndim >= 2
    a, b, c = 3.4445, -4.7750, 2.0315
    X = Gm.to(torch.bfloat16)
    tall = Gm.size(-2) > Gm.size(-1)
    if tall:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.mT
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    if tall:
        X = X.mT
    return X


def muon_scale_factor(n: int, m: int) -> float:
    return 0.2 * max(n, m) ** 0.5


def orthogonalized_updates(params: List[torch.Tensor], updates: List[torch.Tensor], steps: int = 5) -> List[torch.Tensor]:
    """Orthogonalise and scale each update; every entry is a full matrix (or a stack of them)."""
    out = []
    for p, u in zip(params, updates):
        o = zeropower_via_newtonschulz5(u, steps=steps).to(p.dtype)
        out.append(o * muon_scale_factor(u.size(-2), u.size(-1)))
    return out


class Muon(torch.optim.Optimizer):
    """Muon for 2-D hidden weights and stacked 3-D expert weights; pass only Muon-eligible parameters."""

    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, weight_decay: float = 0.1,
                 momentum_dtype: torch.dtype = torch.float32, offload_state: bool = False,
                 max_batch_elems: int = 1 << 28):
        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.momentum_dtype = momentum_dtype
        self.offload_state = offload_state
        self.max_batch_elems = max_batch_elems

    def _state_buf(self, p: torch.Tensor) -> torch.Tensor:
        st = self.state[p]
        if "momentum_buffer" not in st:
            if self.offload_state and p.is_cuda:
                st["momentum_buffer"] = torch.zeros(p.shape, dtype=self.momentum_dtype, device="cpu", pin_memory=True)
            else:
                st["momentum_buffer"] = torch.zeros(p.shape, dtype=self.momentum_dtype, device=p.device)
        return st["momentum_buffer"]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta, lr, wd = group["momentum"], group["lr"], group["weight_decay"]
            for p in group["params"]:
                g = _grad_of(p)
                if g is None or not _owned(p):
                    continue
                self._step_param(p, g, beta, lr, wd)
        return loss

    def _step_param(self, p, g, beta, lr, wd) -> None:
        buf_store = self._state_buf(p)
        offloaded = buf_store.device != p.device
        # stacked experts are processed in slices to bound the fp32 temporaries
        if p.ndim >= 3:
            per = p[0].numel()
            chunk = max(1, self.max_batch_elems // per)
        else:
            chunk = 1
        n_lead = p.shape[0] if p.ndim >= 3 else 1
        for s in range(0, n_lead, chunk):
            sl = slice(s, min(s + chunk, n_lead)) if p.ndim >= 3 else slice(None)
            ps, gs = (p[sl], g[sl]) if p.ndim >= 3 else (p, g)
            bs = buf_store[sl] if p.ndim >= 3 else buf_store
            buf = bs.to(p.device, non_blocking=True).float() if offloaded else bs
            g32 = gs.float()
            if buf.dtype == torch.float32:
                buf.lerp_(g32, 1 - beta)
                upd = g32.lerp(buf, beta)
            else:
                b32 = buf.float().lerp_(g32, 1 - beta)
                buf.copy_(b32)
                upd = g32.lerp(b32, beta)
            if offloaded:
                bs.copy_(buf.to(bs.dtype), non_blocking=True)
            orth = zeropower_via_newtonschulz5(upd, steps=5).to(p.dtype)
            scale = muon_scale_factor(upd.size(-2), upd.size(-1))
            ps.mul_(1 - lr * wd)
            ps.add_(orth, alpha=-lr * scale)


class AdamW(torch.optim.Optimizer):
    """AdamW with fp32 moments over (possibly bf16) owner-sharded parameters."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                g = _grad_of(p)
                if g is None or not _owned(p):
                    continue
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = torch.zeros((), dtype=torch.float32)
                    st["exp_avg"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                    st["exp_avg_sq"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                st["step"] += 1
                t = float(st["step"])
                g32 = g.float()
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.lerp_(g32, 1 - b1)
                v.mul_(b2).addcmul_(g32, g32, value=1 - b2)
                bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
                denom = (v / bc2).sqrt_().add_(eps)
                if p.dtype == torch.float32:
                    p.mul_(1 - lr * wd).addcdiv_(m, denom, value=-lr / bc1)
                else:
                    p32 = p.float().mul_(1 - lr * wd).addcdiv_(m, denom, value=-lr / bc1)
                    p.copy_(p32)
        return loss
