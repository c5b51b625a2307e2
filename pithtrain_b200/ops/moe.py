"""Expert-side MoE compute: routing sort, row gather, SwiGLU, weighted combine, and the fused
expert block with a hand-written backward.

Layout. The expert rank receives ``n`` token rows ``x[n, H]``, their ``k`` routing weights
``w[n, k]`` and local expert ids ``eids[n, k]`` (``-1`` marks a slot whose expert lives on another
rank). :func:`route_sort` counting-sorts the ``n*k`` slots by expert into groups aligned to 16 rows
and returns device-side ``offs[E+1]`` plus the two permutations; all buffers are sized from the
static upper bound ``n*k + 16*E`` so no count is ever read back to the host (the reference syncs
twice per layer here: pithtrain/operators/ep_dispatch.py:630-646,
pithtrain/operators/token_scatter.py:227-264).

:func:`moe_experts` then computes ``partial[t] = sum_j w[t,j] * down_e(act(gate_up_e(x[t])))`` — the
routing weights are applied on the expert rank, so the tensor that travels back is one row per
received token (the reference returns one row per (token, expert) pair and sums at home,
pithtrain/models/qwen3_moe.py:229-245). Its backward never stores the per-slot expert outputs:
the routing-weight gradient is recovered as ``<dgrad_of_down(d_out[t]), act>`` inside the SwiGLU
backward kernel, which also emits the weight-scaled activation consumed by the down-projection
wgrad.
"""

from __future__ import annotations

import os
from typing import Callable, Optional

import torch

from .. import _native
from ..dualpipe.utils import WeightGradStore
from . import gemm as G
from .common import accumulate_grad, sp, use_native

ALIGN = 16


def sorted_capacity(n_slots: int, num_experts: int) -> int:
    """Static row capacity of the expert-sorted layout for ``n_slots`` slots."""
    cap = n_slots + ALIGN * num_experts
    return (cap + 127) // 128 * 128


# ------------------------------------------------------------------------------------------------
# route_sort
# ------------------------------------------------------------------------------------------------
def route_sort_ref(eids: torch.Tensor, num_experts: int, r_cap: int):
    n = eids.numel()
    e = eids.view(-1).long()
    valid = (e >= 0) & (e < num_experts)
    counts = torch.bincount(e[valid], minlength=num_experts)
    padded = (counts + ALIGN - 1) // ALIGN * ALIGN
    offs = torch.zeros(num_experts + 1, dtype=torch.long, device=eids.device)
    offs[1:] = padded.cumsum(0)
    key = torch.where(valid, e, torch.full_like(e, num_experts))
    order = torch.sort(key, stable=True).indices  # slots grouped by expert, slot order inside
    sorted_key = key[order]
    n_valid = int(valid.sum())
    rank_in_group = torch.arange(n, device=eids.device) - torch.cat(
        [torch.zeros(1, dtype=torch.long, device=eids.device), counts.cumsum(0)])[sorted_key.clamp(max=num_experts)]
    row = offs[sorted_key.clamp(max=num_experts - 1)] + rank_in_group
    row_of_slot = torch.full((n,), -1, dtype=torch.int32, device=eids.device)
    slot_of_row = torch.full((r_cap,), -1, dtype=torch.int32, device=eids.device)
    ord_v, row_v = order[:n_valid], row[:n_valid]
    row_of_slot[ord_v] = row_v.int()
    slot_of_row[row_v] = ord_v.int()
    return offs.int(), row_of_slot, slot_of_row


def route_sort(eids: torch.Tensor, num_experts: int, r_cap: Optional[int] = None,
               n_valid: Optional[torch.Tensor] = None):
    """Stable counting sort of slots by expert.

    Returns ``offs[E+1]`` (int32), ``row_of_slot[n]`` (-1 for skipped slots) and ``slot_of_row[r_cap]``
    (-1 for pad rows). ``n_valid`` optionally bounds the slots by a device-side count.
    """
    flat = eids.reshape(-1)
    n = flat.numel()
    if r_cap is None:
        r_cap = sorted_capacity(n, num_experts)
    if not flat.is_cuda:
        if n_valid is not None:
            flat = flat.clone()
            flat[int(n_valid):] = -1
        return route_sort_ref(flat, num_experts, r_cap)
    L = _native.lib()
    flat = flat.int() if flat.dtype != torch.int32 else flat
    flat = flat.contiguous()
    dev = flat.device
    chunks = (n + 511) // 512
    counts = torch.empty((chunks + 1) * num_experts, dtype=torch.int32, device=dev)  # workspace of the chunked sort
    offs = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    row_of_slot = torch.empty(n, dtype=torch.int32, device=dev)
    slot_of_row = torch.empty(r_cap, dtype=torch.int32, device=dev)
    rc = L.pt_route_sort(flat.data_ptr(), None if n_valid is None else n_valid.data_ptr(), n, num_experts,
                         ALIGN, counts.data_ptr(), counts.numel(), offs.data_ptr(), row_of_slot.data_ptr(),
                         slot_of_row.data_ptr(), r_cap, sp())
    _native.check(rc, "pt_route_sort")
    return offs, row_of_slot, slot_of_row


# ------------------------------------------------------------------------------------------------
# gather / combine / swiglu primitives (no autograd; used by the fused block and by other ops)
# ------------------------------------------------------------------------------------------------
def gather_rows(src: torch.Tensor, idx: torch.Tensor, div: int = 1,
                n_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dst[r] = src[idx[r] // div]``, zero rows where ``idx[r] < 0``; rows past ``n_rows`` undefined."""
    R, H = idx.numel(), src.shape[-1]
    if use_native(src) and H % 8 == 0 and src.stride(-1) == 1:
        dst = torch.empty((R, H), dtype=src.dtype, device=src.device)
        rc = _native.lib().pt_gather_rows(src.data_ptr(), idx.data_ptr(), div, dst.data_ptr(),
                                          None if n_rows is None else n_rows.data_ptr(), R, H, src.stride(0), sp())
        _native.check(rc, "pt_gather_rows")
        return dst
    i = idx.long()
    out = src[(i.clamp(min=0) // div)]
    return out * (i >= 0).unsqueeze(-1).to(src.dtype)


def combine_rows(y: torch.Tensor, row_of_slot: torch.Tensor, k: int, w: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = residual[t] + sum_j w[t,j] * y[row_of_slot[t*k+j]]`` skipping negative rows."""
    n = row_of_slot.numel() // k
    H = y.shape[-1]
    if use_native(y) and H % 8 == 0:
        out = torch.empty((n, H), dtype=y.dtype, device=y.device)
        wf = None if w is None else w.float().contiguous()
        rc = _native.lib().pt_combine(y.data_ptr(), row_of_slot.data_ptr(), None if wf is None else wf.data_ptr(),
                                      None if residual is None else residual.contiguous().data_ptr(),
                                      out.data_ptr(), None, n, k, H, sp())
        _native.check(rc, "pt_combine")
        return out
    r = row_of_slot.view(n, k).long()
    rows = y[r.clamp(min=0)].float() * (r >= 0).unsqueeze(-1)
    if w is not None:
        rows = rows * w.float().view(n, k, 1)
    out = rows.sum(1)
    if residual is not None:
        out = out + residual.float()
    return out.to(y.dtype)


def _swiglu_math(g, u, alpha, limit):
    if limit > 0:
        gc = g.clamp(max=limit)
        uc = u.clamp(min=-limit, max=limit)
        return (uc + 1) * gc * torch.sigmoid(alpha * gc)
    return torch.nn.functional.silu(g) * u


def _split_gu(gu, interleaved):
    I = gu.shape[-1] // 2
    if interleaved:
        return gu[..., 0::2], gu[..., 1::2]
    return gu[..., :I], gu[..., I:]


def swiglu_fwd(gu: torch.Tensor, n_rows: Optional[torch.Tensor] = None, interleaved: bool = False,
               alpha: float = 1.0, limit: float = 0.0) -> torch.Tensor:
    R, I = gu.shape[0], gu.shape[1] // 2
    if use_native(gu) and I % 8 == 0:
        act = torch.empty((R, I), dtype=gu.dtype, device=gu.device)
        rc = _native.lib().pt_swiglu_fwd(gu.data_ptr(), act.data_ptr(), None if n_rows is None else n_rows.data_ptr(),
                                         R, I, int(interleaved), float(alpha), float(limit), sp())
        _native.check(rc, "pt_swiglu_fwd")
        return act
    g, u = _split_gu(gu.float(), interleaved)
    return _swiglu_math(g, u, alpha, limit).to(gu.dtype)


def swiglu_bwd(gu: torch.Tensor, dact: torch.Tensor, row_w: Optional[torch.Tensor] = None,
               n_rows: Optional[torch.Tensor] = None, interleaved: bool = False, alpha: float = 1.0,
               limit: float = 0.0, want_act: bool = False, want_dw: bool = False,
               slot_of_row: Optional[torch.Tensor] = None):
    """Returns ``(dgu, act_scaled or None, d_row_w or None)``; see the kernel comment for semantics.

    With ``slot_of_row`` the weights are given per (token, slot) (``row_w`` flat ``[n*k]``) and looked up
    through the row's slot index (a pad row, index -1, has weight 0); ``d_row_w`` is then ``[n*k]`` too.
    """
    R, I = gu.shape[0], gu.shape[1] // 2
    if slot_of_row is not None and not (use_native(gu) and I % 8 == 0):
        w_ext = torch.cat([row_w.reshape(-1).float(), row_w.new_zeros(1, dtype=torch.float32)])
        dgu, act, d_rows = swiglu_bwd(gu, dact, w_ext[slot_of_row.long()], n_rows, interleaved, alpha, limit, want_act, want_dw)
        dw = None
        if d_rows is not None:
            dw = torch.zeros(row_w.numel() + 1, dtype=torch.float32, device=gu.device)
            dw[slot_of_row.long()] = d_rows  # index -1 (pad rows) lands in the spare last entry
            dw = dw[:-1]
        return dgu, act, dw
    if use_native(gu) and I % 8 == 0:
        dgu = torch.empty_like(gu)
        act = torch.empty((R, I), dtype=gu.dtype, device=gu.device) if want_act else None
        n_w = R if slot_of_row is None else row_w.numel()
        dw = torch.zeros(n_w, dtype=torch.float32, device=gu.device) if want_dw else None
        rw = None if row_w is None else row_w.reshape(-1).float().contiguous()
        rc = _native.lib().pt_swiglu_bwd(gu.data_ptr(), dact.contiguous().data_ptr(), None if rw is None else rw.data_ptr(),
                                         dgu.data_ptr(), None if act is None else act.data_ptr(),
                                         None if dw is None else dw.data_ptr(),
                                         None if n_rows is None else n_rows.data_ptr(), R, I, int(interleaved),
                                         float(alpha), float(limit),
                                         None if slot_of_row is None else slot_of_row.data_ptr(), sp())
        _native.check(rc, "pt_swiglu_bwd")
        return dgu, act, dw
    with torch.enable_grad():
        guf = gu.detach().float().requires_grad_()
        g, u = _split_gu(guf, interleaved)
        a = _swiglu_math(g, u, alpha, limit)
        wt = torch.ones(R, device=gu.device) if row_w is None else row_w.float()
        d = dact.float()
        (dguf,) = torch.autograd.grad(a, guf, d * wt[:, None])
    dw = (d * a.detach()).sum(-1) if want_dw else None
    act = (a.detach() * wt[:, None]).to(gu.dtype) if want_act else None
    return dguf.to(gu.dtype), act, dw


def segment_sum(x: torch.Tensor, offs: torch.Tensor, num_groups: int, row_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-group column sums ``[G, H]`` in fp32 of rows ``[offs[g], offs[g+1])`` (bias gradients), each row optionally
    scaled by ``row_w[r]``."""
    # A segmented reduction over the sorted rows: one pass, no atomics, deterministic: one CTA per (group, column slab)
    # in the kernel, ``torch.segment_reduce`` on the CPU. (An ``index_add_`` by group id
    # sends every element through an atomic on one of only ``G x H`` addresses — the pattern the reference measured
    # at about half of the GPU time before its segmented-sum kernel, pithtrain/operators/indexed_bias_add.py:7-13.)
    # Rows at or past ``offs[-1]`` belong to no group and are not read; ``unsafe`` skips the host-side length check.
    H = x.shape[-1]
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and H % 2 == 0 and x.is_contiguous():
        out = torch.empty((num_groups, H), dtype=torch.float32, device=x.device)
        wf = None if row_w is None else row_w.float().contiguous()
        rc = _native.lib().pt_segment_sum(x.data_ptr(), int(x.dtype == torch.float32), _native.ptr(wf),
                                          offs.data_ptr(), num_groups, out.data_ptr(), H, sp())
        _native.check(rc, "pt_segment_sum")
        return out
    xf = x.float() if row_w is None else x.float() * row_w.float()[:, None]
    o = offs[:num_groups + 1].long()
    return torch.segment_reduce(xf, "sum", lengths=o[1:] - o[:-1], axis=0, unsafe=True)


def indexed_bias_add_rows(x: torch.Tensor, bias: torch.Tensor, offs: torch.Tensor, n_rows: Optional[torch.Tensor] = None,
                          inplace: bool = False) -> torch.Tensor:
    """``x[r] + bias[group(r)]`` for expert-sorted rows (groups from ``offs[E+1]``); rows past ``n_rows`` are left
    as they are. One kernel (binary search of the group per row) instead of arange / bucketize / index / add."""
    E, H = bias.shape
    if use_native(x) and bias.dtype == torch.bfloat16 and H % 8 == 0 and x.is_contiguous() and bias.is_contiguous():
        out = x if inplace else torch.empty_like(x)
        rc = _native.lib().pt_indexed_bias_add(x.data_ptr(), bias.data_ptr(), offs.data_ptr(), E, out.data_ptr(),
                                               _native.ptr(n_rows), x.shape[0], H, sp())
        _native.check(rc, "pt_indexed_bias_add")
        return out
    gid = rows_group_id(offs, x.shape[0]).clamp(max=E - 1)
    return x + bias[gid].to(x.dtype)


def rows_group_id(offs: torch.Tensor, R: int) -> torch.Tensor:
    row = torch.arange(R, device=offs.device)
    return torch.bucketize(row, offs[1:].long(), right=True)


# ------------------------------------------------------------------------------------------------
# fused expert block
# ------------------------------------------------------------------------------------------------
# Fuse the expert-order gather into the A-operand load of the first expert GEMM (TMA tile::gather4 in the producer
# warp). Correct (tests/test_gemm_gpu.py) but measured slower end to end than a separate gather pass, so off.
GATHER_IN_GEMM = False


# Weight gradients of an expert block are produced for two micro-batches at a time (one K-grouped launch per weight
# with two operand pairs): a launch reads and rewrites the whole [experts, out, in] gradient buffer, which costs more
# than its FLOPs, so halving the number of passes is worth holding one micro-batch's operands until the next arrives.
# ``flush_pending_expert_wgrads`` (called at the end of every step, before gradients are reduced) runs what is left.
# Off by default: it keeps dY / act / dGU of one extra micro-batch per layer alive; ``TrainingCfg.pair_expert_wgrads``.
PAIR_EXPERT_WGRADS = False
_PENDING_WGRAD: dict = {}


def _run_expert_wgrad(ew: "ExpertWeights", k: int, a, b) -> None:
    dyg, act_s, dgu, x, slot_of_row, offs, n_rows = a
    xs = gather_rows(x, slot_of_row, div=k, n_rows=n_rows)
    if b is None:
        G.grouped_gemm_tn(dyg, act_s, offs, ew.g2(), accumulate=True)
        G.grouped_gemm_tn(dgu, xs, offs, ew.g1(), accumulate=True)
        return
    dyg2, act2, dgu2, x2, sor2, offs2, n2 = b
    xs2 = gather_rows(x2, sor2, div=k, n_rows=n2)
    G.grouped_gemm_tn_pair(dyg, act_s, offs, dyg2, act2, offs2, ew.g2())
    G.grouped_gemm_tn_pair(dgu, xs, offs, dgu2, xs2, offs2, ew.g1())


def flush_pending_expert_wgrads() -> None:
    """Run the weight gradients of micro-batches that found no partner (odd counts, end of the step)."""
    with torch.no_grad():
        while _PENDING_WGRAD:
            _, (ew, k, mine) = _PENDING_WGRAD.popitem()
            _run_expert_wgrad(ew, k, mine, None)


class ExpertWeights:
    """What :func:`moe_experts` needs from the owning module.

    ``w1`` is the fused gate/up projection ``[E, 2I, H]`` (gate rows first, or interleaved), ``w2`` the
    down projection ``[E, H, I]``; ``g1``/``g2`` return the gradient buffers to accumulate into.
    ``b1``/``b2`` are optional per-expert biases (``[E, 2I]``, ``[E, H]``) as parameters.
    """

    def __init__(self, w1, w2, g1: Callable[[], torch.Tensor], g2: Callable[[], torch.Tensor],
                 b1=None, b2=None, interleaved=False, alpha=1.0, limit=0.0):
        self.w1, self.w2, self.g1, self.g2 = w1, w2, g1, g2
        self.b1, self.b2 = b1, b2
        self.interleaved, self.alpha, self.limit = interleaved, alpha, limit


class _MoEExpertsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eids, ew: ExpertWeights, n_valid):
        n, k = eids.shape
        E = ew.w1.shape[0]
        offs, row_of_slot, slot_of_row = route_sort(eids, E, n_valid=(None if n_valid is None else n_valid * k))
        n_rows = offs[E:E + 1]
        from . import fp8_linear as F8
        from .quant import gemm_fp8_nt, quant_rows

        fp8 = F8.eligible(x, ew.w1) and F8.eligible(x, ew.w2)
        if fp8:
            # gather into expert order and quantise in one pass; weights come from the per-step cache
            q1, s1, _, _ = F8.quantized_weight(ew.w1)
            xq, xsc = quant_rows(x, idx=slot_of_row, div=k, n_rows=n_rows)
            gu = gemm_fp8_nt(xq, xsc, q1, s1, offs=offs)
            del xq, xsc
        elif GATHER_IN_GEMM and use_native(x) and x.shape[1] % 64 == 0:
            # the first expert GEMM reads token rows through the index (TMA gather4): the expert-ordered
            # copy of the activations is never materialised
            gu = G.grouped_gemm_nt(x, ew.w1, offs, a_idx=slot_of_row, a_idx_div=k)
        else:
            xs = gather_rows(x, slot_of_row, div=k, n_rows=n_rows)
            gu = G.grouped_gemm_nt(xs, ew.w1, offs)
        if ew.b1 is not None:
            gu = indexed_bias_add_rows(gu, ew.b1.detach(), offs, n_rows, inplace=True)
        act = swiglu_fwd(gu, n_rows, ew.interleaved, ew.alpha, ew.limit)
        if fp8:
            q2, s2, _, _ = F8.quantized_weight(ew.w2)
            aq, asc = quant_rows(act, n_rows=n_rows)
            y = gemm_fp8_nt(aq, asc, q2, s2, offs=offs)
            del aq, asc
        else:
            y = G.grouped_gemm_nt(act, ew.w2, offs)
        if ew.b2 is not None:
            y = indexed_bias_add_rows(y, ew.b2.detach(), offs, n_rows, inplace=True)
        out = combine_rows(y, row_of_slot, k, w=w)
        ctx.save_for_backward(x, w, gu, offs, row_of_slot, slot_of_row)
        ctx.ew = ew
        ctx.k = k
        ctx.fp8 = fp8
        return out

    @staticmethod
    def backward(ctx, d_out):
        x, w, gu, offs, row_of_slot, slot_of_row = ctx.saved_tensors
        ew, k = ctx.ew, ctx.k
        E = ew.w1.shape[0]
        n_rows = offs[E:E + 1]
        d_out = d_out.contiguous()
        dyg = gather_rows(d_out, slot_of_row, div=k, n_rows=n_rows)  # unscaled d_out per sorted row
        if ctx.fp8:
            from . import fp8_linear as F8
            from .quant import gemm_fp8_nt, quant_rows

            _, _, q2t, s2t = F8.quantized_weight(ew.w2)
            dq, dsc = quant_rows(dyg, n_rows=n_rows)
            da = gemm_fp8_nt(dq, dsc, q2t, s2t, offs=offs)
            del dq, dsc
        else:
            da = G.grouped_gemm_nn(dyg, ew.w2, offs)
        plain = ew.b1 is None and ew.b2 is None
        if plain:
            # routing weights and their gradients are looked up / scattered through the slot index in the kernel
            dgu, act_s, d_w_flat = swiglu_bwd(gu, da, w.reshape(-1), n_rows, ew.interleaved, ew.alpha, ew.limit,
                                              want_act=True, want_dw=True, slot_of_row=slot_of_row)
            d_row_w = row_w = None
        else:
            w_ext = torch.cat([w.reshape(-1).float(), w.new_zeros(1, dtype=torch.float32)])
            row_w = w_ext[slot_of_row.long()]  # -1 (pad) picks the appended zero
            dgu, act_s, d_row_w = swiglu_bwd(gu, da, row_w, n_rows, ew.interleaved, ew.alpha, ew.limit,
                                             want_act=True, want_dw=True)
        del da
        if ew.b2 is not None:
            # y = act @ W2.T + b2 ; the routing-weight gradient also sees the bias term
            gid = rows_group_id(offs, gu.shape[0]).clamp(max=E - 1)
            d_row_w = d_row_w + (dyg.float() * ew.b2.detach()[gid].float()).sum(-1)
            accumulate_grad(ew.b2, segment_sum(dyg, offs, E, row_w=row_w))
        if ew.b1 is not None:
            accumulate_grad(ew.b1, segment_sum(dgu, offs, E))
        if plain:
            d_w = d_w_flat.view(w.shape).to(w.dtype)
        else:
            dw_ext = torch.cat([d_row_w, d_row_w.new_zeros(1)])
            d_w = dw_ext[row_of_slot.long()].view(w.shape).to(w.dtype)
        if ctx.fp8:
            _, _, q1t, s1t = F8.quantized_weight(ew.w1)
            gq, gsc = quant_rows(dgu, n_rows=n_rows)
            dxs = gemm_fp8_nt(gq, gsc, q1t, s1t, offs=offs)
            del gq, gsc
        else:
            dxs = G.grouped_gemm_nn(dgu, ew.w1, offs)
        d_x = combine_rows(dxs, row_of_slot, k) if ctx.needs_input_grad[0] else None
        del dxs

        def wgrad_fn(dyg=dyg, act_s=act_s, dgu=dgu, x=x, slot_of_row=slot_of_row, offs=offs, n_rows=n_rows):
            mine = (dyg, act_s, dgu, x, slot_of_row, offs, n_rows)
            if PAIR_EXPERT_WGRADS and use_native(dyg):
                # an expert block is known by its down projection's storage: the owning module builds a new
                # ExpertWeights view on every call
                key = ew.w2.data_ptr()
                other = _PENDING_WGRAD.pop(key, None)
                if other is None:
                    # wait for the next micro-batch of this expert block: both share one pass over the gradients
                    _PENDING_WGRAD[key] = (ew, k, mine)
                    return
                _run_expert_wgrad(ew, k, other[2], mine)
            else:
                _run_expert_wgrad(ew, k, mine, None)

        if WeightGradStore.enabled:
            WeightGradStore.put(wgrad_fn)
        else:
            wgrad_fn()
        return d_x, d_w, None, None, None


def moe_experts(x: torch.Tensor, w: torch.Tensor, eids: torch.Tensor, ew: ExpertWeights,
                n_valid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Weighted expert outputs for received tokens: ``out[t] = sum_j w[t,j] * expert_{eids[t,j]}(x[t])``."""
    if not x.requires_grad and torch.is_grad_enabled():
        x = x.detach().requires_grad_()
    return _MoEExpertsFn.apply(x.contiguous(), w, eids, ew, n_valid)


def moe_experts_ref(x, w, eids, w1, w2, b1=None, b2=None, interleaved=False, alpha=1.0, limit=0.0):
    """Plain-autograd per-expert loop, the oracle for :func:`moe_experts`."""
    n, k = eids.shape
    out = torch.zeros_like(x, dtype=torch.float32)
    for e in range(w1.shape[0]):
        tok, slot = torch.where(eids == e)
        if tok.numel() == 0:
            continue
        xe = x[tok].float()
        gu = xe @ w1[e].float().t()
        if b1 is not None:
            gu = gu + b1[e].float()
        g, u = _split_gu(gu, interleaved)
        a = _swiglu_math(g, u, alpha, limit)
        y = a @ w2[e].float().t()
        if b2 is not None:
            y = y + b2[e].float()
        out.index_add_(0, tok, y * w[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)
