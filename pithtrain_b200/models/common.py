"""Building blocks shared by the model families: config access, rotary tables (plain and YaRN),
the gate/router module, expert containers with fused storage, the MoE block that implements the
stage-1/3/5 split, and the base class that turns a list of decoder layers into a pipeline chunk.
"""

from __future__ import annotations

import math
from typing import Any, Callable, Optional, Tuple

import torch
import torch.nn as nn

from ..contexts import distributed
from ..dualpipe.dualpipev import layer_partition
from ..dualpipe.execution import ChunkRecord, model_forward
from ..modules.load_balance import MoELoadBalanceLossInjector, MoELoadBalanceLossTracker
from ..ops import gemm as G
from ..ops.embedding import Embedding
from ..ops.linear import FusedWeights, Linear, fused_linear, linear
from ..ops.moe import ExpertWeights, moe_experts, moe_experts_ref
from ..ops.norm import RMSNorm, rmsnorm_ref
from ..ops.router import router_topk, router_topk_ref
from ..parallel import ep as ep_mod
from .interface import RoutingInfo


# ------------------------------------------------------------------------------------------------
# config helpers
# ------------------------------------------------------------------------------------------------
def cfg_get(config: Any, name: str, default: Any = None) -> Any:
    if isinstance(config, dict):
        return config.get(name, default)
    return getattr(config, name, default)


def rope_theta_of(config: Any) -> float:
    """``rope_theta`` wherever the config spells it (top level, ``rope_scaling`` or ``rope_parameters``)."""
    for holder in ("rope_parameters", "rope_scaling"):
        d = cfg_get(config, holder)
        if isinstance(d, dict) and d.get("rope_theta") is not None:
            return float(d["rope_theta"])
    v = cfg_get(config, "rope_theta")
    return float(v) if v is not None else 10000.0


def rope_scaling_of(config: Any) -> Optional[dict]:
    for holder in ("rope_scaling", "rope_parameters"):
        d = cfg_get(config, holder)
        if isinstance(d, dict) and (d.get("rope_type", d.get("type")) not in (None, "default")):
            return d
    return None


def stage_of_phase(phase: int) -> Tuple[int, int]:
    """(stage_index, stage_count) of local chunk ``phase`` (0, 1) or the whole model (-1)."""
    if phase == -1:
        return 0, 1
    count = distributed.pp_size * 2
    if phase == 0:
        return distributed.pp_rank, count
    if phase == 1:
        return count - 1 - distributed.pp_rank, count
    raise ValueError(f"phase must be 0, 1, or -1, got {phase}")


# ------------------------------------------------------------------------------------------------
# rotary embeddings
# ------------------------------------------------------------------------------------------------
def yarn_find_correction_dim(num_rotations, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rotations * 2 * math.pi))) / (2 * math.log(base))


def yarn_inv_freq(dim: int, base: float, factor: float, original_max_pos: int, beta_fast: float = 32.0,
                  beta_slow: float = 1.0, truncate: bool = True) -> torch.Tensor:
    """YaRN frequency blend between interpolated and extrapolated RoPE frequencies."""
    pos_freqs = base ** (torch.arange(0, dim, 2, dtype=torch.float32, device="cpu") / dim)
    extrap, interp = 1.0 / pos_freqs, 1.0 / (factor * pos_freqs)
    low = yarn_find_correction_dim(beta_fast, dim, base, original_max_pos)
    high = yarn_find_correction_dim(beta_slow, dim, base, original_max_pos)
    if truncate:
        low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float32, device="cpu") - low) / (high - low)).clamp(0, 1)
    extrap_mask = 1.0 - ramp
    return interp * (1 - extrap_mask) + extrap * extrap_mask


class RotaryEmbedding(nn.Module):
    """cos/sin tables ``[max_pos, dim]`` (``cat(freqs, freqs)`` layout), built in fp32 and stored in
    ``table_dtype`` (bf16 in the reference: pithtrain/models/qwen3_moe.py:35-39). ``attn_scale``
    (YaRN ``mscale``) is folded into both tables."""

    def __init__(self, dim: int, max_pos: int, base: float, inv_freq: Optional[torch.Tensor] = None,
                 attn_scale: float = 1.0, table_dtype: torch.dtype = torch.bfloat16, device=None):
        super().__init__()
        if inv_freq is None:
            inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32, device="cpu") / dim))
        t = torch.arange(max_pos, dtype=torch.float32, device="cpu")
        freqs = torch.outer(t, inv_freq.float().cpu())
        emb = torch.cat((freqs, freqs), dim=-1)
        self.dim = dim
        device = device if device is not None else distributed.device
        self.register_buffer("cos", (emb.cos() * attn_scale).to(table_dtype).to(device), persistent=False)
        self.register_buffer("sin", (emb.sin() * attn_scale).to(table_dtype).to(device), persistent=False)

    def forward(self, S: int):
        return self.cos[:S], self.sin[:S]


def zigzag_positions(S_local: int, cp_size: int, cp_rank: int, device) -> torch.Tensor:
    """Global positions of this rank's two zigzag blocks (front block r, mirrored block 2cp-1-r)."""
    block = S_local // 2
    front = cp_rank * block
    back = (2 * cp_size - cp_rank - 1) * block
    return torch.cat([torch.arange(front, front + block, device=device), torch.arange(back, back + block, device=device)])


def packed_positions(S: int, cu_seqlens: torch.Tensor) -> torch.Tensor:
    starts = cu_seqlens[:-1].long()
    lengths = (cu_seqlens[1:] - cu_seqlens[:-1]).long()
    return torch.arange(S, device=cu_seqlens.device) - torch.repeat_interleave(starts, lengths, output_size=S)


class RotaryPos:
    """What ``forward_posemb`` hands to the layers: the tables plus per-token positions."""

    __slots__ = ("cos", "sin", "positions", "S")

    def __init__(self, cos, sin, positions, S):
        self.cos, self.sin, self.positions, self.S = cos, sin, positions, S

    def gathered(self, n_tokens: int):
        """(cos, sin) rows per token ``[n_tokens, dim]`` for code paths that want them materialised."""
        if self.positions is None:
            pos = torch.arange(n_tokens, device=self.cos.device) % self.S
        else:
            pos = self.positions.long()
            if pos.numel() != n_tokens:
                pos = pos.repeat(n_tokens // pos.numel())
        return self.cos[pos], self.sin[pos]

    def token_positions(self, n_tokens: int) -> Optional[torch.Tensor]:
        if self.positions is None:
            return None
        pos = self.positions
        if pos.numel() != n_tokens:
            pos = pos.repeat(n_tokens // pos.numel())
        return pos.int()


# ------------------------------------------------------------------------------------------------
# router
# ------------------------------------------------------------------------------------------------
class Gate(nn.Module):
    """MoE router: linear -> (softmax, top-k) in either order -> optional renorm / scale.

    ``load_balance_loss_fn`` and ``router_replay`` are attached by ``setup_model``
    (pithtrain/modules/training.py:439-460 in the reference does the same).
    """

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, mode: str = "softmax_topk",
                 norm_topk_prob: bool = False, scale: float = 1.0, bias: bool = False,
                 fp32_logits: bool = False, device=None, dtype=None):
        super().__init__()
        self.num_experts, self.num_experts_per_tok = num_experts, top_k
        self.mode, self.norm_topk_prob, self.scale, self.fp32_logits = mode, norm_topk_prob, scale, fp32_logits
        self.load_balance_loss_fn: Optional[Callable] = None
        self.router_replay: Optional[Callable] = None
        self.weight = nn.Parameter(torch.empty((num_experts, hidden_size), device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(num_experts, device=device, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def logits(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.fp32_logits:
            return torch.nn.functional.linear(tokens.float(), self.weight.float(),
                                              None if self.bias is None else self.bias.float())
        return linear(tokens, self.weight, self.bias, fp8=False)

    def forward(self, tokens: torch.Tensor, reference: bool = False):
        """Returns ``(topk_idx[m,k] int32, topk_weight[m,k] fp32, lb_loss or None)``."""
        logits = self.logits(tokens)
        fn = router_topk_ref if reference else router_topk
        if self.router_replay is not None and self.mode == "softmax_topk":
            scores = logits.float().softmax(-1)
            idx = self.router_replay(torch.topk(scores, self.num_experts_per_tok, dim=-1).indices)
            w = scores.gather(-1, idx.long())
            if self.norm_topk_prob:
                w = w / w.sum(-1, keepdim=True)
            w, idx = w * self.scale, idx.int()
        else:
            w, idx, scores = fn(logits, self.num_experts_per_tok, self.mode, self.norm_topk_prob, self.scale)
        lb_loss = None
        if self.load_balance_loss_fn is not None:
            if scores is None:
                scores = logits.float().softmax(-1)
            lb_loss = self.load_balance_loss_fn(scores, idx, self.num_experts, self.num_experts_per_tok)
            # weight the injected gradient by the token count so the trainer's 1/num_tokens scale
            # normalises it like the token-summed cross-entropy
            w = MoELoadBalanceLossInjector.apply(w, lb_loss * w.shape[0])
        return idx, w, lb_loss


# ------------------------------------------------------------------------------------------------
# experts
# ------------------------------------------------------------------------------------------------
class _ExpertProj(nn.Module):
    """Holder of one stacked expert weight ``[E, out, in]`` under the name ``<proj>.weight``."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, device=None, dtype=None):
        super().__init__()
        self.num_groups, self.in_features, self.out_features = num_experts, in_features, out_features
        self.weight = nn.Parameter(torch.empty((num_experts, out_features, in_features), device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=0.02)


class SwiGLUExperts(nn.Module):
    """``down(silu(gate(x)) * up(x))`` experts with separate ``gate_proj/up_proj/down_proj`` parameters
    (checkpoint names of Qwen3-MoE and DeepSeek-V2) whose gate and up stacks share one
    ``[E, 2, I, H]`` storage so the first grouped GEMM sees a fused ``[E, 2I, H]`` operand."""

    def __init__(self, num_experts: int, hidden_size: int, intermediate_size: int, device=None, dtype=None):
        super().__init__()
        self.gate_proj = _ExpertProj(num_experts, hidden_size, intermediate_size, device, dtype)
        self.up_proj = _ExpertProj(num_experts, hidden_size, intermediate_size, device, dtype)
        self.down_proj = _ExpertProj(num_experts, intermediate_size, hidden_size, device, dtype)
        self.fused_gate_up = FusedWeights([self.gate_proj.weight, self.up_proj.weight], layout="pair")

    def expert_weights(self) -> ExpertWeights:
        from ..ops.common import grad_buffer

        w1 = self.fused_gate_up.ensure()
        return ExpertWeights(w1, self.down_proj.weight, self.fused_gate_up.grad,
                             lambda: grad_buffer(self.down_proj.weight))

    def reference(self, x, w, eids):
        w1 = torch.cat([self.gate_proj.weight, self.up_proj.weight], dim=1)
        return moe_experts_ref(x, w, eids, w1, self.down_proj.weight)


class MoEBlock(nn.Module):
    """Gate + local experts with the stage-1/3/5 split and expert-parallel bookkeeping."""

    def __init__(self, gate: Gate, experts: nn.Module, num_experts: int, top_k: int, gate_attr: str = "gate"):
        super().__init__()
        self._gate_attr = gate_attr
        self.num_experts, self.num_experts_per_tok = num_experts, top_k
        self.ep_size, self.ep_rank = distributed.ep_size, distributed.ep_rank
        assert num_experts % self.ep_size == 0
        self.experts_per_rank = num_experts // self.ep_size
        setattr(self, gate_attr, gate)
        self.experts = experts

    @property
    def router_module(self) -> Gate:
        return getattr(self, self._gate_attr)

    # stage 1 tail
    def route(self, tokens: torch.Tensor) -> RoutingInfo:
        idx, w, lb_loss = self.router_module(tokens)
        if lb_loss is not None:
            MoELoadBalanceLossTracker.add(lb_loss)
        plan = None
        ex = ep_mod.current()
        if ex is not None:
            plan = ex.plan(idx, self.num_experts)
        return RoutingInfo(topk_weight=w, topk_idx=idx, plan=plan, lb_loss=lb_loss)

    # stage 3
    def experts_forward(self, tokens: torch.Tensor, weights: torch.Tensor, routing: RoutingInfo) -> torch.Tensor:
        if routing.plan is None:
            eids, n_valid = routing.topk_idx, None
        else:
            eids, n_valid = routing.plan.recv_eids, routing.plan.n_recv_dev
        return moe_experts(tokens, weights, eids, self.experts.expert_weights(), n_valid=n_valid)

    # stage 5 head
    def finish(self, outs: torch.Tensor, routing: RoutingInfo) -> torch.Tensor:
        if routing.plan is None or getattr(routing.plan, "reduced", False):
            return outs
        return ep_mod.home_reduce(outs, routing.plan)

    def reference_forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """Single-rank oracle (all experts local)."""
        idx, w, lb_loss = self.router_module(tokens, reference=True)
        if lb_loss is not None:
            MoELoadBalanceLossTracker.add(lb_loss)
        return self.experts.reference(tokens, w, idx)


class DenseMLP(nn.Module):
    """SwiGLU MLP with fused gate/up GEMM (dense layers, shared experts)."""

    def __init__(self, hidden_size: int, intermediate_size: int, device=None, dtype=None):
        super().__init__()
        self.gate_proj = Linear(hidden_size, intermediate_size, bias=False, device=device, dtype=dtype)
        self.up_proj = Linear(hidden_size, intermediate_size, bias=False, device=device, dtype=dtype)
        self.down_proj = Linear(intermediate_size, hidden_size, bias=False, device=device, dtype=dtype)
        self.fused_gate_up = FusedWeights([self.gate_proj.weight, self.up_proj.weight], layout="rows")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops.activations import swiglu

        gu = fused_linear(x, self.fused_gate_up)
        return self.down_proj(swiglu(gu))

    def reference(self, x: torch.Tensor) -> torch.Tensor:
        F = torch.nn.functional
        return F.linear(F.silu(F.linear(x, self.gate_proj.weight)) * F.linear(x, self.up_proj.weight), self.down_proj.weight)


# ------------------------------------------------------------------------------------------------
# pipeline chunk base class
# ------------------------------------------------------------------------------------------------
class PipelineChunk(nn.Module):
    """One model chunk: optional embedding (first stage), a slice of decoder layers, optional final
    norm + lm_head (last stage). Subclasses provide ``build_layer`` and ``build_rotary``."""

    def __init__(self, config: Any, phase: int):
        super().__init__()
        self.config = config
        self.stage_index, self.stage_count = stage_of_phase(phase)
        self.chunk_record: Optional[ChunkRecord] = None
        H, V = cfg_get(config, "hidden_size"), cfg_get(config, "vocab_size")
        self.rotary_emb = self.build_rotary(config)
        self.embed_tokens, self.norm, self.lm_head = None, None, None
        if self.stage_index == 0:
            self.embed_tokens = Embedding(V, H)
        if self.stage_index == self.stage_count - 1:
            self.norm = self.build_norm(config)
            self.lm_head = Linear(H, V, bias=False)
            self.lm_head.fp8 = False  # the vocabulary projection stays bf16
        ids = layer_partition(cfg_get(config, "num_hidden_layers"), self.stage_count, self.stage_index)
        self.layers = nn.ModuleDict({str(i): self.build_layer(config, i) for i in ids})

    # hooks
    def build_layer(self, config, idx: int) -> nn.Module:
        raise NotImplementedError

    def build_rotary(self, config) -> nn.Module:
        raise NotImplementedError

    def build_norm(self, config) -> nn.Module:
        return RMSNorm(cfg_get(config, "hidden_size"), eps=cfg_get(config, "rms_norm_eps", 1e-6))

    supports_cp = True
    supports_packed = True

    # protocol
    def forward_posemb(self, S: int, cu_seqlens: Optional[torch.Tensor] = None) -> RotaryPos:
        dev = self.rotary_emb.cos.device
        if cu_seqlens is not None:
            if not self.supports_packed:
                raise NotImplementedError(f"{type(self).__name__} does not support packed sequences")
            return RotaryPos(self.rotary_emb.cos, self.rotary_emb.sin, packed_positions(S, cu_seqlens), S)
        if distributed.cp_size > 1:
            if not self.supports_cp:
                raise NotImplementedError(f"{type(self).__name__} does not support context parallelism")
            pos = zigzag_positions(S, distributed.cp_size, distributed.cp_rank, dev)
            return RotaryPos(self.rotary_emb.cos, self.rotary_emb.sin, pos, S)
        return RotaryPos(self.rotary_emb.cos, self.rotary_emb.sin, None, S)

    def forward_prolog(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.embed_tokens(hidden_states)

    def forward_epilog(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.lm_head(self.norm(hidden_states))

    def forward(self, hidden_states: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.chunk_record is None:
            self.chunk_record = ChunkRecord(len(self.layers))
        return model_forward(self, hidden_states, self.chunk_record, cu_seqlens)

    def reference_forward(self, hidden_states: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.stage_index == 0:
            hidden_states = torch.nn.functional.embedding(hidden_states, self.embed_tokens.weight)
        rotary = self.forward_posemb(hidden_states.shape[1], cu_seqlens)
        for layer in self.layers.values():
            hidden_states = layer.reference_forward(hidden_states, rotary, cu_seqlens)
        if self.stage_index == self.stage_count - 1:
            h = rmsnorm_ref(hidden_states, self.norm.weight, self.norm.eps, zero_centered=self.norm.zero_centered)
            hidden_states = torch.nn.functional.linear(h, self.lm_head.weight)
        return hidden_states
