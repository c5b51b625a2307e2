"""Activation memory of one decoder layer for one micro-batch, stage by stage.

Each entry names a tensor this framework's hand-written autograd functions keep between the forward
and the backward of a micro-batch (pithtrain_b200/ops/*.py, pithtrain_b200/models/common.py). Tensors are
grouped by the stage that creates them, and flagged ``wgrad`` when a deferred weight-gradient
closure still needs them after the activation backward ran (zero-bubble B/W split). The
reference's estimator does the same bookkeeping for torch.compile-saved tensors
(tools/memory_estimator/activation_profile.py:121-231 of the reference).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List

from .model_profile import ModelDims, ParallelCfg


@dataclass
class TokenCounts:
    T: int  # tokens of one micro-batch on this rank
    recv: int  # de-duplicated rows received by this rank's experts
    sorted_rows: int  # (row, expert) pairs after the expert sort, incl. alignment padding
    recv_capacity: int  # rows of the receive buffers (what is actually allocated)


def token_counts(dims: ModelDims, par: ParallelCfg, imbalance: float = 1.0) -> TokenCounts:
    T, ep, k = par.tokens_per_microbatch, par.ep, dims.k
    hit = 1.0 - ((ep - 1) / ep) ** k if ep > 1 else 1.0
    recv = int(ep * T * hit * imbalance) if ep > 1 else T
    pairs = int(T * k * imbalance)
    worst = ep * T
    if par.ep_backend == "fused" and ep > 1:
        cap = worst  # exact worst case unless a capacity factor is opted into
        if par.capacity_factor is not None:
            want = int(par.capacity_factor * ep * T * hit) + T
            cap = min(worst, (want + 127) // 128 * 128)
    else:
        cap = recv
    # the expert-side buffers (sorted row index, gate/up output) are allocated for every received row hitting k local
    # experts: nothing is read back to the host to size them by what actually arrived
    sorted_rows = (cap * k if ep > 1 else pairs) + 16 * (dims.E // ep)
    return TokenCounts(T=T, recv=min(recv, worst), sorted_rows=sorted_rows, recv_capacity=cap)


@dataclass
class Saved:
    name: str
    stage: int
    nbytes: int
    wgrad: bool = False  # still needed by a deferred weight-gradient closure


def layer_saved(dims: ModelDims, par: ParallelCfg, idx: int, tc: TokenCounts) -> List[Saved]:
    H, T = dims.H, tc.T
    ls = dims.layer_shape(idx)
    out: List[Saved] = []
    add = lambda *a, **kw: out.append(Saved(*a, **kw))
    bf = 2
    # ---------------------------------------------------------------- stage 1: attention + router
    add("hidden_in", 1, T * H * bf)
    add("input_norm.rstd", 1, T * 4)
    add("attn.x_normed", 1, T * H * bf, wgrad=True)
    ak = ls.attn_kind
    if ak in ("gqa", "gated_gqa"):
        qw = dims.nh * dims.d_qk * (2 if ak == "gated_gqa" else 1)
        kvw = 2 * dims.nkv * dims.d_qk
        add("attn.qkv", 1, T * (qw + kvw) * bf)
        add("attn.q_k_roped", 1, T * (dims.nh + dims.nkv) * dims.d_qk * bf)
        add("attn.out", 1, T * dims.nh * dims.d_qk * bf, wgrad=True)
        add("attn.lse", 1, T * dims.nh * 4)
        if ak == "gated_gqa":
            add("attn.gated_out", 1, T * dims.nh * dims.d_qk * bf, wgrad=True)
    elif ak == "mla":
        add("attn.q", 1, T * dims.nh * dims.d_qk * bf)
        add("attn.kv_latent", 1, T * (dims.kv_lora + dims.d_rope) * bf * 2, wgrad=True)
        add("attn.kv_expanded", 1, T * dims.nh * (dims.d_qk - dims.d_rope + dims.d_v) * bf)
        add("attn.q_k_roped", 1, 2 * T * dims.nh * dims.d_qk * bf)
        add("attn.out", 1, T * dims.nh * dims.d_v * bf, wgrad=True)
        add("attn.lse", 1, T * dims.nh * 4)
    else:  # gated delta net
        kd, vd = dims.lin_nk * dims.lin_dk, dims.lin_nv * dims.lin_dv
        add("lin.qkvz", 1, T * (2 * kd + 2 * vd) * bf)
        add("lin.conv_out", 1, T * (2 * kd + vd) * bf)
        add("lin.qk_normed", 1, 2 * T * dims.lin_nv * dims.lin_dk * bf)
        add("lin.gates", 1, 2 * T * dims.lin_nv * 4)
        add("lin.chunk_states", 1, (T // 64 + 1) * dims.lin_nv * dims.lin_dk * dims.lin_dv * 4)
        add("lin.out", 1, 2 * T * vd * bf, wgrad=True)
    add("residual_mid", 1, T * H * bf)
    add("post_norm.rstd", 1, T * 4)
    add("mlp.tokens", 1, T * H * bf, wgrad=True)
    if ls.kind == "dense":
        add("mlp.gate_up", 1, T * 2 * dims.I_dense * bf)
        add("mlp.act", 1, T * dims.I_dense * bf, wgrad=True)
        return out
    add("router.scores", 1, T * dims.E * 4)
    add("router.topk", 1, T * dims.k * 8)
    if ls.shared_params:
        add("shared.gate_up", 1, T * 2 * dims.I_shared * bf)
        add("shared.act", 1, T * dims.I_shared * bf, wgrad=True)
    add("ep.plan", 1, T * par.ep * 4 + tc.recv_capacity * dims.k * 4 if par.ep > 1 else 0)
    # ---------------------------------------------------------------- stage 2/3: dispatch + experts
    if par.ep > 1:
        add("ep.recv_x", 2, tc.recv_capacity * H * bf, wgrad=True)
        add("ep.recv_w", 2, tc.recv_capacity * dims.k * 8)
    add("experts.sort_index", 3, (tc.sorted_rows + tc.recv * dims.k) * 4, wgrad=True)
    add("experts.gate_up", 3, tc.sorted_rows * 2 * dims.I_moe * bf)
    # ---------------------------------------------------------------- stage 4/5: combine
    if par.ep > 1:
        add("ep.partial_out", 4, tc.recv_capacity * H * bf)
    return out


def layer_bytes(dims: ModelDims, par: ParallelCfg, idx: int, tc: TokenCounts) -> tuple:
    """(bytes held from F to B, bytes that survive B until the deferred W)."""
    s = layer_saved(dims, par, idx, tc)
    total = sum(x.nbytes for x in s)
    # a deferred weight gradient needs the GEMM input (flagged) and the matching output gradient,
    # which is about as large as the input of the next op; count the flagged tensors twice
    held = 2 * sum(x.nbytes for x in s if x.wgrad)
    return total, min(held, total)


def edge_bytes(dims: ModelDims, par: ParallelCfg, first: bool, last: bool, tc: TokenCounts) -> int:
    """Prolog/epilog extras: token ids, and on the last stage the final norm input + logits (the
    cross-entropy kernel overwrites the logits with their gradient in place)."""
    n = 0
    if first:
        n += tc.T * 8
    if last:
        n += tc.T * dims.H * 2 * 2 + tc.T * dims.V * 2 + tc.T * 8
    return n
