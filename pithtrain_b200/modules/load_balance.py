"""MoE load-balance losses, their gradient injector and the benchmark router replay.

All three losses have the Switch form ``coef * E * sum_i f_i * P_i`` with ``f`` the fraction of
routed slots per expert and ``P`` the mean router probability; they differ in what ``f`` is counted
over: the micro-batch, the global batch (counts all-reduced over dp×ep and accumulated over
micro-batches), or each sequence (counts all-reduced over cp). Public names and semantics follow
pithtrain/modules/load_balance.py:21-274 of the reference.
"""

from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def expert_token_counts(idx_flat: torch.Tensor, n_bins: int) -> torch.Tensor:
    """Histogram without the host sync of ``torch.bincount`` on CUDA (ids must lie in [0, n_bins))."""
    out = torch.zeros(n_bins, dtype=torch.float32, device=idx_flat.device)
    out.scatter_add_(0, idx_flat.long(), torch.ones((), device=idx_flat.device).expand(idx_flat.numel()))
    return out


class MoELoadBalanceLossInjector(torch.autograd.Function):
    """Identity on ``output`` that routes a gradient of one into ``lb_loss`` during backward."""

    @staticmethod
    def forward(ctx, output: torch.Tensor, lb_loss: torch.Tensor) -> torch.Tensor:
        ctx.save_for_backward(lb_loss)
        return output.view_as(output)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        (lb_loss,) = ctx.saved_tensors
        return grad_output, torch.ones_like(lb_loss)


class MicroBatchLoadBalanceLoss:
    def __init__(self, lb_coef: float) -> None:
        self.lb_coef = lb_coef

    def __call__(self, scores, topk_idx, num_experts: int, top_k: int) -> torch.Tensor:
        n = scores.shape[0]
        f = expert_token_counts(topk_idx.reshape(-1), num_experts) / (n * top_k)
        return self.lb_coef * num_experts * torch.dot(f.to(scores.dtype), scores.mean(dim=0))

    def reset(self) -> None:
        pass


class GlobalBatchLoadBalanceLoss:
    def __init__(self, lb_coef: float, process_group=None) -> None:
        self.lb_coef = lb_coef
        self.process_group = process_group
        self.group_size = dist.get_world_size(process_group) if process_group is not None else 1
        self._counts: Optional[torch.Tensor] = None
        self._total = 0

    def init_buffers(self, num_experts: int, device) -> None:
        if self._counts is None:
            self._counts = torch.zeros(num_experts, dtype=torch.float32, device=device)

    def __call__(self, scores, topk_idx, num_experts: int, top_k: int) -> torch.Tensor:
        self.init_buffers(num_experts, scores.device)
        counts = expert_token_counts(topk_idx.reshape(-1), num_experts)
        if self.process_group is not None:
            dist.all_reduce(counts, group=self.process_group)
        self._counts.add_(counts)
        self._total += scores.shape[0] * top_k * self.group_size
        f = self._counts / self._total
        return self.lb_coef * num_experts * torch.dot(f.to(scores.dtype), scores.mean(dim=0))

    def reset(self) -> None:
        if self._counts is not None:
            self._counts.zero_()
        self._total = 0


class SequenceLevelLoadBalanceLoss:
    def __init__(self, lb_coef: float, sequence_length: int, cp_group=None) -> None:
        self.lb_coef = lb_coef
        self.sequence_length = sequence_length
        self.cp_group = cp_group
        self.cp_size = dist.get_world_size(cp_group) if cp_group is not None else 1

    def __call__(self, scores, topk_idx, num_experts: int, top_k: int) -> torch.Tensor:
        S = self.sequence_length
        B = scores.shape[0] // S
        offs = (torch.arange(B, device=topk_idx.device) * num_experts).view(B, 1)
        flat = topk_idx.view(B, -1).long() + offs
        counts = expert_token_counts(flat.reshape(-1), B * num_experts).view(B, num_experts)
        if self.cp_group is not None:
            dist.all_reduce(counts, group=self.cp_group)
        f = counts / (S * self.cp_size * top_k)
        p = scores.view(B, S, num_experts).mean(dim=1)
        return self.lb_coef * ((f.to(scores.dtype) * p).sum(dim=1) * num_experts).mean()

    def reset(self) -> None:
        pass


class MoELoadBalanceLossTracker:
    """Collects the per-layer losses of a step for logging and resets stateful loss objects."""

    instances: List = []
    losses: List = []

    @classmethod
    def register(cls, instance) -> None:
        cls.instances.append(instance)

    @classmethod
    def reset(cls) -> None:
        for inst in cls.instances:
            inst.reset()

    @classmethod
    def add(cls, loss: torch.Tensor) -> None:
        cls.losses.append(loss.detach())

    @classmethod
    def get_total_count_and_clear(cls) -> Tuple[float, int]:
        if not cls.losses:
            return 0.0, 0
        total = float(torch.stack(cls.losses).sum().item())
        count = len(cls.losses)
        cls.losses.clear()
        return total, count


def make_load_balance_loss_fn(lb_type: str, lb_coef: float, process_group=None, sequence_length: int = 0,
                              cp_group=None):
    """Callable ``(scores, topk_idx, num_experts, top_k) -> loss`` for a gate, registered with the tracker."""
    if lb_type == "micro-batch":
        loss = MicroBatchLoadBalanceLoss(lb_coef)
    elif lb_type == "global-batch":
        loss = GlobalBatchLoadBalanceLoss(lb_coef, process_group)
    elif lb_type == "sequence":
        loss = SequenceLevelLoadBalanceLoss(lb_coef, sequence_length, cp_group)
    else:
        raise ValueError(f"Unknown moe_load_balance_type: {lb_type!r}")
    MoELoadBalanceLossTracker.register(loss)
    return loss


def force_balance(num_experts: int) -> Callable[[torch.Tensor], torch.Tensor]:
    """Benchmark-only router replay: token ``t`` slot ``j`` goes to expert ``(t + j*E/k) mod E``."""

    def replay(topk_idx: torch.Tensor) -> torch.Tensor:
        n, k = topk_idx.shape
        stride = num_experts // k
        t = torch.arange(n, device=topk_idx.device).unsqueeze(1)
        j = torch.arange(k, device=topk_idx.device).unsqueeze(0)
        return ((t + j * stride) % num_experts).to(topk_idx.dtype)

    return replay
