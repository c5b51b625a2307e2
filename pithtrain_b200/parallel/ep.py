"""Expert-parallel exchange with token de-duplication in both directions.

Dispatch sends each token once per destination rank that owns at least one of its top-k experts,
together with its routing weights and the local expert ids of its slots there (-1 for slots that
belong to other ranks). The expert rank applies the routing weights itself and pre-sums a token's
expert outputs, so combine returns one row per *dispatched* row — the same volume as dispatch —
instead of one row per (token, expert) pair as in the reference
(pithtrain/operators/ep_dispatch.py:579-676, pithtrain/models/qwen3_moe.py:240-245). Backward of each
exchange is the opposite exchange over the same plan.

Index math of a plan (``m`` local tokens, ``ep`` ranks, ``k`` slots per token):

* ``sent[t, g]``            token t has a slot on rank g
* ``send_token_idx[r]``     token of send row r (rows ordered by destination, then token)
* ``token_send_pos[t, g]``  send row of (t, g), or -1
* ``send_eids[r, j]``       local expert id of slot j on the row's destination, or -1

Two transports implement :class:`Exchange`: :class:`CollectiveExchange` (``all_to_all_single`` over
NCCL or gloo — the baseline path, which has to read the receive counts back to the host) and the
fused peer-memory transport in :mod:`pithtrain_b200.parallel.ep_fused`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops.moe import combine_rows, gather_rows

_CURRENT = None


def current():
    """The process-wide exchange (``None`` when ``ep_size == 1``)."""
    return _CURRENT


def set_current(exchange) -> None:
    global _CURRENT
    _CURRENT = exchange


@dataclass
class DispatchPlan:
    m: int
    k: int
    ep: int
    send_token_idx: torch.Tensor  # [n_send] int32
    token_send_pos: torch.Tensor  # [m, ep] int32
    send_eids: torch.Tensor  # [n_send, k] int32
    send_counts: List[int]
    recv_counts: List[int]
    recv_eids: Optional[torch.Tensor] = None  # [n_recv, k] int32, filled by the plan exchange
    n_recv_dev: Optional[torch.Tensor] = None  # device-side count (fused transport)

    @property
    def n_send(self) -> int:
        return int(self.send_token_idx.numel())

    @property
    def n_recv(self) -> int:
        return int(sum(self.recv_counts))


def build_send_side(topk_idx: torch.Tensor, num_experts: int, ep: int):
    """Sender-side index math, pure tensor ops (also the CPU oracle of the fused route-plan kernel).

    Returns ``(send_token_idx, token_send_pos, send_eids, send_counts[ep] tensor)``.
    """
    m, k = topk_idx.shape
    epr = num_experts // ep
    idx = topk_idx.long()
    dest = idx // epr  # [m, k]
    ranks = torch.arange(ep, device=idx.device)
    sent = (dest.unsqueeze(-1) == ranks).any(dim=1)  # [m, ep]
    send_counts = sent.sum(0)
    offsets = torch.cumsum(send_counts, 0) - send_counts
    pos_in_chunk = torch.cumsum(sent.long(), 0) - 1
    token_send_pos = torch.where(sent, pos_in_chunk + offsets.unsqueeze(0), torch.full_like(pos_in_chunk, -1))
    g_of_row, t_of_row = torch.nonzero(sent.t(), as_tuple=True)
    local = idx[t_of_row] - (g_of_row * epr).unsqueeze(-1)
    on_dest = dest[t_of_row] == g_of_row.unsqueeze(-1)
    send_eids = torch.where(on_dest, local, torch.full_like(local, -1))
    return t_of_row.int(), token_send_pos.int(), send_eids.int(), send_counts


class _A2A(torch.autograd.Function):
    """all_to_all_single whose backward is the exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.splits = (in_splits, out_splits)
        ctx.group = group
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        in_splits, out_splits = ctx.splits
        out = g.new_empty((sum(in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), in_splits, out_splits, group=ctx.group)
        return out, None, None, None


class _GatherSend(torch.autograd.Function):
    """rows[r] = x[send_token_idx[r]]; backward sums a token's rows over its destinations."""

    @staticmethod
    def forward(ctx, x, plan: DispatchPlan):
        ctx.plan = plan
        return gather_rows(x, plan.send_token_idx)

    @staticmethod
    def backward(ctx, g):
        p = ctx.plan
        return combine_rows(g.contiguous(), p.token_send_pos.reshape(-1), p.ep), None


class _HomeReduce(torch.autograd.Function):
    """out[t] = sum over destinations of the partial row that came back for (t, dest)."""

    @staticmethod
    def forward(ctx, back, plan: DispatchPlan):
        ctx.plan = plan
        return combine_rows(back.contiguous(), plan.token_send_pos.reshape(-1), plan.ep)

    @staticmethod
    def backward(ctx, g):
        return gather_rows(g.contiguous(), ctx.plan.send_token_idx), None


def home_reduce(back: torch.Tensor, plan: DispatchPlan) -> torch.Tensor:
    return _HomeReduce.apply(back, plan)


class Exchange:
    """Interface of an expert-parallel transport."""

    ep: int

    def plan(self, topk_idx: torch.Tensor, num_experts: int) -> DispatchPlan: ...

    def dispatch(self, x: torch.Tensor, w: torch.Tensor, plan: DispatchPlan) -> Tuple[torch.Tensor, torch.Tensor]: ...

    def combine(self, partial: torch.Tensor, plan: DispatchPlan) -> torch.Tensor: ...


class CollectiveExchange(Exchange):
    """Baseline transport: ``all_to_all_single`` on the ep process group (NCCL or gloo)."""

    def __init__(self, group, ep_size: int, ep_rank: int) -> None:
        self.group, self.ep, self.rank = group, ep_size, ep_rank

    def plan(self, topk_idx: torch.Tensor, num_experts: int) -> DispatchPlan:
        m, k = topk_idx.shape
        send_token_idx, token_send_pos, send_eids, send_counts = build_send_side(topk_idx, num_experts, self.ep)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()  # host read-back: the price of this transport
        recv_eids = send_eids.new_empty((sum(rc), k))
        dist.all_to_all_single(recv_eids, send_eids.contiguous(), rc, sc, group=self.group)
        return DispatchPlan(m=m, k=k, ep=self.ep, send_token_idx=send_token_idx, token_send_pos=token_send_pos,
                            send_eids=send_eids, send_counts=sc, recv_counts=rc, recv_eids=recv_eids)

    def dispatch(self, x, w, plan):
        rows = _GatherSend.apply(x, plan)
        w_rows = w[plan.send_token_idx.long()]
        recv_x = _A2A.apply(rows, plan.send_counts, plan.recv_counts, self.group)
        recv_w = _A2A.apply(w_rows, plan.send_counts, plan.recv_counts, self.group)
        return recv_x, recv_w

    def combine(self, partial, plan):
        return _A2A.apply(partial, plan.recv_counts, plan.send_counts, self.group)


def _fused_transport_usable(d) -> bool:
    """True when every rank of the expert group sits on this node with peer access to the others.

    The expert axis is the innermost mesh axis, so a group is ``ep_size`` consecutive ranks; it stays
    inside a node when the node's rank count is a multiple of ``ep_size``. The ranks vote (MIN over the
    group) so that all of them pick the same transport.
    """
    if torch.device(d.device).type != "cuda":
        return False
    local_world = max(int(getattr(d, "local_world_size", 1) or 1), 1)
    ok = d.ep_size <= local_world and local_world % d.ep_size == 0
    if ok:
        from .. import _native

        me = torch.device(d.device).index or 0
        base = me - d.ep_rank
        L = _native.lib()
        ok = all(L.pt_can_access_peer(me, base + r) == 1 for r in range(d.ep_size) if base + r != me)
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=d.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=d.ep_group)
    return bool(flag.item())


def setup_exchange(backend: str = "auto", capacity_factor: float | None = None):
    """Create the process-wide exchange from the distributed context (call after setup_distributed)."""
    from ..contexts import distributed

    if distributed.ep_size == 1:
        set_current(None)
        return None
    if backend == "auto":
        backend = "fused" if _fused_transport_usable(distributed) else "nccl"
    if backend == "fused":
        from .ep_fused import FusedExchange

        ex = FusedExchange(distributed.ep_group, distributed.ep_size, distributed.ep_rank, capacity_factor)
    else:
        ex = CollectiveExchange(distributed.ep_group, distributed.ep_size, distributed.ep_rank)
    set_current(ex)
    return ex
