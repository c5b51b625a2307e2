"""Context-parallel attention over a zigzag-sharded sequence.

The sequence is cut into ``2*cp`` blocks and rank ``r`` holds blocks ``r`` and ``2cp-1-r`` (front and
back), which balances causal work. Every rank needs the keys/values of all earlier blocks: the KV
payload of each rank visits every other rank (ring over NCCL/gloo p2p, or direct pulls from the
owner's symmetric buffer), and each visit contributes a partial ``(out, lse)`` that is merged with a
running log-sum-exp. Which (query block, key block) pairs interact, and with which mask, is decided
from global block indices, so the same code serves plain causal attention, sliding windows
(GPT-OSS) and learned sinks (added to the denominator once, at the end). The backward pass visits
the payloads again, recomputes each partial from the *global* ``lse`` and accumulates key/value
gradients in fp32 buffers that travel with the payload back to its owner.

The payload is generic: plain ``(k, v)``, or the MLA latent ``(normed_kv, k_pe)`` that is expanded
by ``kv_b_proj`` on arrival (576 instead of 5120 values per token on the wire); the expansion's
weight gradient accumulates locally. Reference counterpart: pithtrain/operators/ring_attention.py
(:28-48 schedule, :112-140 merge, :143-280 zigzag forward/backward, :428-708 MLA latent ring); the
reference refuses sinks and windows under context parallelism (pithtrain/models/gpt_oss.py:361-362).
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..contexts import distributed

NEG_INF = float("-inf")


# ------------------------------------------------------------------------------------------------
# block-level attention with an explicit log-sum-exp (math path; works on CPU and GPU)
# ------------------------------------------------------------------------------------------------
def _expand_kv(k: torch.Tensor, Hq: int) -> torch.Tensor:
    Hkv = k.shape[2]
    return k if Hkv == Hq else k.repeat_interleave(Hq // Hkv, dim=2)


def geometric_mask(Sq: int, Sk: int, causal: bool, q_off: int, window_left: Optional[int], device) -> Optional[torch.Tensor]:
    """Boolean ``[Sq, Sk]`` of a block pair whose query row ``r`` sits at position ``q_off + r`` relative to key 0:
    causal and sliding-window visibility; None when every key is visible."""
    if not causal and window_left is None:
        return None
    qp = torch.arange(Sq, device=device).unsqueeze(1) + q_off
    kp = torch.arange(Sk, device=device).unsqueeze(0)
    m = torch.ones(Sq, Sk, dtype=torch.bool, device=device)
    if causal:
        m &= kp <= qp
    if window_left is not None:
        m &= kp >= qp - window_left
    return m


def _own_kernels(q, k, v) -> bool:
    from . import attention_native as N

    return N.supported(q, k, v, True, None, None, None)


def block_fwd(q, k, v, scale: float, causal: bool = False, q_off: int = 0, window_left: Optional[int] = None
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Partial attention of ``q[B,Sq,Hq,D]`` against ``k,v[B,Sk,Hkv,*]``: ``out[B,Sq,Hq,Dv]`` and fp32
    ``lse[B,Hq,Sq]`` (``-inf`` for rows that see no key). Query row ``r`` sits at position ``q_off + r`` relative to
    key 0; ``causal`` and ``window_left`` restrict visibility from there. bf16 blocks on a GPU run on the tcgen05
    forward kernel (csrc/attention.cu), everything else on the fp32 math below."""
    if _own_kernels(q, k, v):
        from . import attention_native as N

        row_lo = N.row_lower_bounds(q.shape[0], q.shape[1], q_off, window_left, None, q.device)
        return N.forward(q, k, v, scale, causal, q_off, row_lo, None)
    mask = geometric_mask(q.shape[1], k.shape[1], causal, q_off, window_left, q.device)
    Hq = q.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = _expand_kv(k, Hq).float().permute(0, 2, 1, 3)
    vf = _expand_kv(v, Hq).float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, NEG_INF)
    lse = torch.logsumexp(s, dim=-1)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - safe.unsqueeze(-1))
    out = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return out, lse


def block_bwd(do, q, k, v, out, lse, scale: float, causal: bool = False, q_off: int = 0, window_left: Optional[int] = None):
    """Gradients of one partial given the *global* ``out``/``lse`` (flash-attention backward math); the tcgen05
    backward kernel (csrc/attention_bwd.cu) for the head dims it covers."""
    from . import attention_native as N

    if _own_kernels(q, k, v) and (q.shape[-1], v.shape[-1]) in N._BWD_DIMS and q.shape[1] % 4 == 0:
        row_lo = N.row_lower_bounds(q.shape[0], q.shape[1], q_off, window_left, None, q.device)
        dq, dk, dv, _ = N.backward(do.to(q.dtype), q, k, v, out.to(q.dtype), lse, scale, causal, q_off, row_lo)
        return dq, dk, dv
    mask = geometric_mask(q.shape[1], k.shape[1], causal, q_off, window_left, q.device)
    Hq, Hkv = q.shape[2], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = _expand_kv(k, Hq).float().permute(0, 2, 1, 3)
    vf = _expand_kv(v, Hq).float().permute(0, 2, 1, 3)
    dof = do.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, NEG_INF)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - safe.unsqueeze(-1))
    delta = (dof * out.float().permute(0, 2, 1, 3)).sum(-1, keepdim=True)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf).permute(0, 2, 1, 3)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    B, _, Sk, _ = dk.shape
    if g > 1:
        dk = dk.view(B, Hkv, g, Sk, -1).sum(2)
        dv = dv.view(B, Hkv, g, Sk, -1).sum(2)
    return dq, dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3)


def merge_partial_math(out: torch.Tensor, lse: torch.Tensor, o_p: torch.Tensor, lse_p: torch.Tensor):
    """Tensor-op restatement of the merge (fp32): the CPU path and the oracle of the kernel."""
    new = torch.logaddexp(lse, lse_p)
    safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
    w_old = torch.exp(lse - safe).permute(0, 2, 1).unsqueeze(-1)
    w_new = torch.exp(lse_p - safe).permute(0, 2, 1).unsqueeze(-1)
    return out * w_old + o_p.float() * w_new, new


MERGE_KERNEL = True  # GPU: one pass of csrc/merge.cu instead of the eight tensor ops of merge_partial_math


def merge_partial(out: Optional[torch.Tensor], lse: Optional[torch.Tensor], o_p: torch.Tensor, lse_p: torch.Tensor):
    """Fold a partial ``(o_p [B, S, H, D], lse_p [B, H, S])`` into the running fp32 ``(out, lse)``.

    The running ``out`` is updated in place on the kernel path (it is a private accumulator of the ring loop).
    Counterpart in the reference: the ``combine_partial`` step of pithtrain/operators/ring_attention.py.
    """
    if out is None:
        return o_p.float(), lse_p
    B, S, H, D = o_p.shape
    if (MERGE_KERNEL and out.is_cuda and out.dtype == torch.float32 and out.is_contiguous() and lse.is_contiguous()
            and lse_p.is_contiguous() and lse.dtype == torch.float32 and lse_p.dtype == torch.float32
            and o_p.dtype in (torch.bfloat16, torch.float32) and D % 4 == 0 and o_p.stride(3) == 1
            and o_p.stride(2) == D and o_p.stride(0) == S * o_p.stride(1) and o_p.stride(1) % 4 == 0
            and o_p.data_ptr() % 16 == 0):
        from .. import _native

        new = torch.empty_like(lse)
        rc = _native.lib().pt_merge_partial(out.data_ptr(), lse.data_ptr(), o_p.data_ptr(), int(o_p.dtype == torch.float32),
                                            lse_p.data_ptr(), new.data_ptr(), B, S, H, D, o_p.stride(1), _native.stream_ptr())
        _native.check(rc, "pt_merge_partial")
        return out, new
    return merge_partial_math(out, lse, o_p, lse_p)


# ------------------------------------------------------------------------------------------------
# zigzag geometry
# ------------------------------------------------------------------------------------------------
def zigzag_blocks(cp: int, r: int) -> Tuple[int, int]:
    return r, 2 * cp - 1 - r


def pair_relation(qb: int, kb: int, block: int, window_left: Optional[int]) -> str:
    """How query block ``qb`` sees key block ``kb``: "skip", "full" or "mask"."""
    if kb > qb:
        return "skip"
    if window_left is not None:
        # closest pair of positions: first query of qb vs last key of kb
        if qb * block - (kb * block + block - 1) > window_left:
            return "skip"
        return "mask"
    return "mask" if kb == qb else "full"


# ------------------------------------------------------------------------------------------------
# payload transport (ring over the cp process group)
# ------------------------------------------------------------------------------------------------
def _rotate(tensors: Sequence[torch.Tensor], group, cp: int, rank: int):
    """Post send-to-next / recv-from-previous for every tensor; returns (received, requests)."""
    nxt, prv = (rank + 1) % cp, (rank - 1) % cp
    g_nxt = dist.get_global_rank(group, nxt) if group is not None else nxt
    g_prv = dist.get_global_rank(group, prv) if group is not None else prv
    recv = [torch.empty_like(t) for t in tensors]
    ops = []
    for t, r in zip(tensors, recv):
        ops.append(dist.P2POp(dist.isend, t.contiguous(), g_nxt, group))
        ops.append(dist.P2POp(dist.irecv, r, g_prv, group))
    return recv, dist.batch_isend_irecv(ops)


def _wait(reqs) -> None:
    for r in reqs:
        r.wait()


class _NcclRing:
    """Payload moves one hop per step around the ring (``batch_isend_irecv``)."""

    def __init__(self, payload, group, cp: int, rank: int):
        self.cur, self.group, self.cp, self.rank = payload, group, cp, rank
        self.nxt, self.reqs = None, []

    def begin_step(self, i: int):
        if i < self.cp - 1:
            self.nxt, self.reqs = _rotate(self.cur, self.group, self.cp, self.rank)
        return self.cur

    def end_step(self, i: int) -> None:
        _wait(self.reqs)
        self.reqs = []
        if self.nxt is not None:
            self.cur, self.nxt = self.nxt, None

    def finish(self) -> None:
        pass


class _PeerPull:
    """Payload is published once in symmetric memory; step ``i`` reads rank ``rank - i`` directly, with the
    next step's block being fetched on a side stream meanwhile (pithtrain_b200/parallel/cp_fused.py)."""

    def __init__(self, kind: str, payload, group, cp: int, rank: int, with_grads: bool, in_place: bool = False):
        from ..parallel.cp_fused import get_exchange

        self.cp, self.rank, self.local = cp, rank, payload
        self.ex = get_exchange(kind, group, cp, rank, payload, with_grads)
        self.epoch = self.ex.publish(payload)
        self.pending = None
        self.in_place = in_place  # remote blocks are read where they were published: nothing is copied ahead

    def begin_step(self, i: int):
        if i == 0:
            cur = self.local
        else:
            cur, ev = self.pending
            torch.cuda.current_stream().wait_event(ev)
        more = i < self.cp - 1 and not self.in_place
        self.pending = self.ex.pull((self.rank - i - 1) % self.cp, self.epoch) if more else None
        return cur

    def end_step(self, i: int) -> None:
        pass

    def finish(self) -> None:
        self.ex.finish(self.epoch)


_PULL_OK: dict = {}


def _peer_pull_usable(group, cp: int, device) -> bool:
    """Decided once per (group, device): the vote inside is a collective."""
    key = (id(group), cp, str(device))
    if key not in _PULL_OK:
        from ..parallel import cp_fused

        _PULL_OK[key] = cp_fused.usable(group, cp, device)
    return _PULL_OK[key]


# Forward steps read a peer's published K/V where it lies (the attention kernel's TMA loads cross NVLink) instead of
# copying the block first.
IN_PLACE_REMOTE_BLOCKS = True


def _in_place_blocks_usable(q: torch.Tensor, payload, expand, window_left: Optional[int]) -> bool:
    """Remote K/V blocks can be consumed where their owner published them in the case the kernel's pointer form covers:
    plain K and V (no latent to expand), no window, one sequence per micro-batch, head dim 64 or 128, bf16."""
    if not IN_PLACE_REMOTE_BLOCKS or expand is not None or window_left is not None or len(payload) != 2:
        return False
    k, v = payload
    B, S2, Hq, D = q.shape
    return (B == 1 and D in (64, 128) and k.shape[-1] == D and v.shape[-1] == D and q.dtype == torch.bfloat16
            and k.dtype == torch.bfloat16 and Hq % k.shape[2] == 0)


def _pairs(cp: int, rank: int, src: int, block: int, window_left: Optional[int]):
    """(q half, k half, relation, q block id, k block id) for local queries vs the payload of ``src``."""
    out = []
    for qi, qb in enumerate(zigzag_blocks(cp, rank)):
        for ki, kb in enumerate(zigzag_blocks(cp, src)):
            rel = pair_relation(qb, kb, block, window_left)
            if rel != "skip":
                out.append((qi, ki, rel, qb, kb))
    return out


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, sinks, scale, window_left, group, cp, rank, expand, n_payload, *rest):
        payload = list(rest[:n_payload])
        params = list(rest[n_payload:])
        B, S2, Hq, _ = q.shape
        block = S2 // 2
        dev = q.device
        q_halves = (q[:, :block], q[:, block:])
        outs: List[Optional[torch.Tensor]] = [None, None]
        lses: List[Optional[torch.Tensor]] = [None, None]
        start = [t.detach() for t in payload]
        pull = q.is_cuda and cp > 1 and _peer_pull_usable(group, cp, dev)
        in_place = pull and _in_place_blocks_usable(q, start, expand, window_left)
        ring = _PeerPull("fwd", start, group, cp, rank, False, in_place) if pull else _NcclRing(start, group, cp, rank)
        for i in range(cp):
            src = (rank - i) % cp
            if in_place and i > 0:
                # the attention kernel's own TMA loads fetch the remote block over NVLink while it computes
                from . import attention_native as N

                Hkv, D = start[0].shape[2], start[0].shape[3]
                half = block * Hkv * D * start[0].element_size()
                ring.ex.wait_ready(src, ring.epoch)
                for qi, ki, rel, qb, kb in _pairs(cp, rank, src, block, None):
                    assert rel == "full"  # without a window, blocks of other ranks are entirely visible or entirely not
                    o_p, lse_p = N.block_from_pointers(q_halves[qi], ring.ex.peer_ptr(src, ring.epoch, 0) + ki * half,
                                                       ring.ex.peer_ptr(src, ring.epoch, 1) + ki * half, block, Hkv, scale)
                    outs[qi], lses[qi] = merge_partial(outs[qi], lses[qi], o_p, lse_p)
                continue
            cur = ring.begin_step(i)
            with torch.no_grad():
                k, v = expand(cur, params) if expand is not None else (cur[0], cur[1])
                k_halves, v_halves = (k[:, :block], k[:, block:]), (v[:, :block], v[:, block:])
                for qi, ki, rel, qb, kb in _pairs(cp, rank, src, block, window_left):
                    o_p, lse_p = block_fwd(q_halves[qi], k_halves[ki], v_halves[ki], scale, rel == "mask",
                                           (qb - kb) * block, window_left)
                    outs[qi], lses[qi] = merge_partial(outs[qi], lses[qi], o_p, lse_p)
            ring.end_step(i)
        ring.finish()
        out = torch.cat(outs, dim=1)
        lse = torch.cat(lses, dim=2)
        if sinks is not None:
            tot = torch.logaddexp(lse, sinks.float().view(1, Hq, 1))
            out = out * torch.exp(lse - tot).permute(0, 2, 1).unsqueeze(-1)
            lse = tot
        out = out.to(q.dtype)
        ctx.save_for_backward(q, out, lse, sinks, *payload, *params)
        ctx.cfg = (scale, window_left, group, cp, rank, expand, n_payload)
        ctx.param_refs = params
        return out

    @staticmethod
    def backward(ctx, do):
        scale, window_left, group, cp, rank, expand, n_payload = ctx.cfg
        q, out, lse, sinks = ctx.saved_tensors[:4]
        payload = list(ctx.saved_tensors[4:4 + n_payload])
        params = list(ctx.saved_tensors[4 + n_payload:])
        B, S2, Hq, _ = q.shape
        block = S2 // 2
        dev = q.device
        halves = lambda t, dim=1: (t.narrow(dim, 0, block), t.narrow(dim, block, block))
        q_h, do_h, out_h, lse_h = halves(q), halves(do), halves(out), halves(lse, 2)
        dq = [torch.zeros(B, block, Hq, q.shape[-1], dtype=torch.float32, device=dev) for _ in range(2)]
        start = [t.detach() for t in payload]
        pull = q.is_cuda and cp > 1 and _peer_pull_usable(group, cp, dev)
        ring = _PeerPull("bwd", start, group, cp, rank, True) if pull else _NcclRing(start, group, cp, rank)
        dacc = [torch.zeros(t.shape, dtype=torch.float32, device=dev) for t in payload]
        dparams = [torch.zeros(p.shape, dtype=torch.float32, device=dev) for p in params]
        local_part = None
        for i in range(cp):
            src = (rank - i) % cp
            cur = ring.begin_step(i)
            if pull:
                dacc = [torch.zeros(t.shape, dtype=torch.float32, device=dev) for t in payload]
            with torch.enable_grad():
                leaves = [t.detach().requires_grad_(t.is_floating_point()) for t in cur]
                p_leaves = [p.detach().requires_grad_() for p in params]
                k, v = expand(leaves, p_leaves) if expand is not None else (leaves[0], leaves[1])
            dk = torch.zeros(k.shape, dtype=torch.float32, device=dev)
            dv = torch.zeros(v.shape, dtype=torch.float32, device=dev)
            with torch.no_grad():
                k_h, v_h = halves(k.detach()), halves(v.detach())
                dk_h, dv_h = halves(dk), halves(dv)
                for qi, ki, rel, qb, kb in _pairs(cp, rank, src, block, window_left):
                    dq_p, dk_p, dv_p = block_bwd(do_h[qi], q_h[qi], k_h[ki], v_h[ki], out_h[qi], lse_h[qi], scale,
                                                 rel == "mask", (qb - kb) * block, window_left)
                    dq[qi] += dq_p
                    dk_h[ki].add_(dk_p)
                    dv_h[ki].add_(dv_p)
            if expand is None:
                dacc[0] += dk
                dacc[1] += dv
            else:
                grads = torch.autograd.grad((k, v), leaves + p_leaves, (dk.to(k.dtype), dv.to(v.dtype)), allow_unused=True)
                for j in range(n_payload):
                    if grads[j] is not None:
                        dacc[j] += grads[j].float()
                for j, g in enumerate(grads[n_payload:]):
                    if g is not None:
                        dparams[j] += g.float()
            ring.end_step(i)
            if pull:
                # the partial goes straight to the owner of the block (own block: kept)
                if i == 0:
                    local_part = dacc
                else:
                    ring.ex.push_grad(src, ring.epoch, dacc)
            else:
                # the gradient accumulators follow their payload around the ring and end at its owner
                dacc, reqs2 = _rotate(dacc, group, cp, rank)
                _wait(reqs2)
        ring.finish()
        if pull:
            dacc = ring.ex.collect_grads(ring.epoch, local_part)
        d_sinks = None
        if sinks is not None:
            delta = (do.float() * out.float()).sum(-1).permute(0, 2, 1)  # [B,Hq,S]
            d_sinks = -(torch.exp(sinks.float().view(1, Hq, 1) - lse) * delta).sum((0, 2)).to(sinks.dtype)
        from .common import accumulate_grad

        for p, g in zip(ctx.param_refs, dparams):
            accumulate_grad(p, g)
        d_payload = [g.to(t.dtype) if t.is_floating_point() else None for g, t in zip(dacc, payload)]
        return (torch.cat(dq, dim=1).to(q.dtype), d_sinks, None, None, None, None, None, None, None,
                *d_payload, *([None] * len(params)))


def _cp():
    return distributed.cp_group, distributed.cp_size, distributed.cp_rank


def ring_attention_func(q, k, v, softmax_scale: Optional[float] = None, window_left: Optional[int] = None,
                        sinks: Optional[torch.Tensor] = None, cp_group=None, cp_size: Optional[int] = None,
                        cp_rank: Optional[int] = None) -> torch.Tensor:
    """Causal attention for zigzag-sharded ``q,k,v [B, S/cp, H, D]``; returns ``[B, S/cp, Hq, Dv]``."""
    g, n, r = _cp()
    group = cp_group if cp_group is not None else g
    cp = cp_size if cp_size is not None else n
    rank = cp_rank if cp_rank is not None else r
    scale = softmax_scale if softmax_scale is not None else q.shape[-1] ** -0.5
    return _RingAttention.apply(q, sinks, scale, window_left, group, cp, rank, None, 2, k, v)


def _mla_expand(num_heads: int, nope: int, v_dim: int):
    def expand(payload, params):
        normed_kv, k_pe = payload
        (w,) = params
        B, S, _ = normed_kv.shape
        kv = torch.nn.functional.linear(normed_kv, w).view(B, S, num_heads, nope + v_dim)
        k_nope, v = torch.split(kv, [nope, v_dim], dim=-1)
        k = torch.cat([k_nope, k_pe.expand(-1, -1, num_heads, -1)], dim=-1)
        return k, v

    return expand


def mla_ring_attention_func(q_nope, q_pe, normed_kv, k_pe, kv_b_proj, sm_scale: float, qk_nope_head_dim: int,
                            v_head_dim: int, cp_group=None) -> torch.Tensor:
    """MLA under context parallelism: the ring carries the latent ``(normed_kv, k_pe)`` and every rank
    expands it with ``kv_b_proj`` on arrival; ``kv_b_proj.weight`` gets its gradient accumulated."""
    g, cp, rank = _cp()
    group = cp_group if cp_group is not None else g
    q = torch.cat([q_nope, q_pe], dim=-1)
    w = kv_b_proj.weight if hasattr(kv_b_proj, "weight") else kv_b_proj
    expand = _mla_expand(q.shape[2], qk_nope_head_dim, v_head_dim)
    return _RingAttention.apply(q, None, sm_scale, None, group, cp, rank, expand, 2, normed_kv, k_pe, w)
