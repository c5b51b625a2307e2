"""DeepSeek-V2 / DeepSeek-V2-Lite: multi-head latent attention (MLA), fp32 softmax router with
optional group-limited top-k, shared experts, leading dense layers.

Math specification: pithtrain/models/deepseek_v2.py:26-88 (YaRN tables), :146-171 (gate),
:213-277 (MLA), :285-347 (layer stages) of the reference. Shared experts are evaluated in stage 1
on the local tokens and folded into the residual, so only routed-expert traffic crosses ranks.
Under context parallelism the ring carries the compressed latent (``kv_lora_rank + rope`` values
per token) instead of per-head keys and values.
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..contexts import distributed
from ..modules.load_balance import MoELoadBalanceLossInjector
from ..ops.attention import attention, attention_ref
from ..ops.linear import FusedWeights, Linear, fused_linear
from ..ops.norm import RMSNorm, rmsnorm_ref
from ..ops.rope import apply_rope_ref
from .common import (DenseMLP, Gate, MoEBlock, PipelineChunk, RotaryEmbedding, RotaryPos, SwiGLUExperts, cfg_get,
                     rope_scaling_of, rope_theta_of, yarn_inv_freq)


def yarn_mscale(factor: float, mscale: float) -> float:
    return 1.0 if factor <= 1 else 0.1 * mscale * math.log(factor) + 1.0


class DeepSeekV2MoEGate(Gate):
    """fp32 logits -> softmax -> (group-limited) top-k -> ``* routed_scaling_factor``; no renormalisation."""

    def __init__(self, config: Any):
        super().__init__(cfg_get(config, "hidden_size"), cfg_get(config, "n_routed_experts"),
                         cfg_get(config, "num_experts_per_tok"), mode="softmax_topk", norm_topk_prob=False,
                         scale=float(cfg_get(config, "routed_scaling_factor", 1.0)), fp32_logits=True)
        self.topk_method = cfg_get(config, "topk_method", "greedy")
        self.num_group = cfg_get(config, "n_group", 1) or 1
        self.topk_group = cfg_get(config, "topk_group", 1) or 1
        self.n_routed_experts = self.num_experts
        self.top_k = self.num_experts_per_tok

    def forward(self, tokens: torch.Tensor, reference: bool = False):
        if self.topk_method != "group_limited_greedy":
            return super().forward(tokens, reference)
        logits = self.logits(tokens)
        scores = logits.softmax(dim=-1, dtype=torch.float32)
        n = scores.shape[0]
        group_scores = scores.view(n, self.num_group, -1).max(dim=-1).values
        group_idx = torch.topk(group_scores, k=self.topk_group, dim=-1, sorted=False)[1]
        group_mask = torch.zeros_like(group_scores).scatter_(1, group_idx, 1.0)
        score_mask = group_mask.unsqueeze(-1).expand(n, self.num_group, self.num_experts // self.num_group).reshape(n, -1)
        masked = scores.masked_fill(~score_mask.bool(), 0.0)
        w, idx = torch.topk(masked, k=self.top_k, dim=-1, sorted=False)
        if self.router_replay is not None:
            idx = self.router_replay(idx)
            w = masked.gather(-1, idx.long())
        w = w * self.scale
        lb_loss = None
        if self.load_balance_loss_fn is not None:
            lb_loss = self.load_balance_loss_fn(masked, idx, self.num_experts, self.top_k)
            w = MoELoadBalanceLossInjector.apply(w, lb_loss * w.shape[0])
        return idx.int(), w, lb_loss


class DeepSeekV2MoE(MoEBlock):
    def __init__(self, config: Any):
        E, k = cfg_get(config, "n_routed_experts"), cfg_get(config, "num_experts_per_tok")
        H, I = cfg_get(config, "hidden_size"), cfg_get(config, "moe_intermediate_size")
        super().__init__(DeepSeekV2MoEGate(config), SwiGLUExperts(E // distributed.ep_size, H, I), E, k)
        self.n_routed_experts = E
        n_shared = cfg_get(config, "n_shared_experts", 0) or 0
        self.shared_experts = DenseMLP(H, I * n_shared) if n_shared > 0 else None

    def reference_forward(self, tokens: torch.Tensor) -> torch.Tensor:
        y = super().reference_forward(tokens)
        if self.shared_experts is not None:
            y = y + self.shared_experts.reference(tokens)
        return y


class DeepSeekV2MLP(DenseMLP):
    def __init__(self, config: Any, intermediate_size: Optional[int] = None):
        super().__init__(cfg_get(config, "hidden_size"), intermediate_size or cfg_get(config, "intermediate_size"))

    def reference_forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.reference(x)


def interleaved_to_half(x: torch.Tensor) -> torch.Tensor:
    """Reorder the last dim from (x0,y0,x1,y1,..) pairs to (x0,x1,..,y0,y1,..) halves."""
    *lead, D = x.shape
    return x.view(*lead, D // 2, 2).transpose(-1, -2).reshape(*lead, D)


class DeepSeekV2Attention(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        H = cfg_get(config, "hidden_size")
        self.num_heads = cfg_get(config, "num_attention_heads")
        self.qk_rope_head_dim = cfg_get(config, "qk_rope_head_dim")
        self.qk_nope_head_dim = cfg_get(config, "qk_nope_head_dim")
        self.kv_lora_rank = cfg_get(config, "kv_lora_rank")
        self.v_head_dim = cfg_get(config, "v_head_dim")
        self.q_head_dim = self.qk_nope_head_dim + self.qk_rope_head_dim
        self.q_lora_rank = cfg_get(config, "q_lora_rank")
        eps = cfg_get(config, "rms_norm_eps", 1e-6)
        self.eps = eps
        if self.q_lora_rank is None:
            self.q_proj = Linear(H, self.num_heads * self.q_head_dim, bias=False)
        else:
            self.q_a_proj = Linear(H, self.q_lora_rank, bias=False)
            self.q_a_layernorm = RMSNorm(self.q_lora_rank, eps=eps)
            self.q_b_proj = Linear(self.q_lora_rank, self.num_heads * self.q_head_dim, bias=False)
        self.kv_a_proj_with_mqa = Linear(H, self.kv_lora_rank + self.qk_rope_head_dim, bias=False)
        self.kv_a_layernorm = RMSNorm(self.kv_lora_rank, eps=eps)
        self.kv_b_proj = Linear(self.kv_lora_rank, self.num_heads * (self.qk_nope_head_dim + self.v_head_dim), bias=False)
        self.o_proj = Linear(self.num_heads * self.v_head_dim, H, bias=False)
        self.softmax_scale = self.q_head_dim ** -0.5
        first = self.q_proj.weight if self.q_lora_rank is None else self.q_a_proj.weight
        # hidden -> (q | latent kv) in one GEMM
        self.fused_in = FusedWeights([first, self.kv_a_proj_with_mqa.weight], layout="rows")

    def _project(self, x: torch.Tensor, reference: bool):
        B, S, H = x.shape
        if reference:
            first = self.q_proj if self.q_lora_rank is None else self.q_a_proj
            q = F.linear(x, first.weight)
            ckv = F.linear(x, self.kv_a_proj_with_mqa.weight)
        else:
            both = fused_linear(x.view(B * S, H), self.fused_in).view(B, S, -1)
            n_first = self.fused_in.params[0].shape[0]
            q, ckv = both[..., :n_first], both[..., n_first:]
        if self.q_lora_rank is not None:
            if reference:
                q = F.linear(rmsnorm_ref(q, self.q_a_layernorm.weight, self.eps), self.q_b_proj.weight)
            else:
                q = self.q_b_proj(self.q_a_layernorm(q.contiguous()))
        q = q.reshape(B, S, self.num_heads, self.q_head_dim)
        q_nope, q_pe = torch.split(q, [self.qk_nope_head_dim, self.qk_rope_head_dim], dim=-1)
        compressed, k_pe = torch.split(ckv, [self.kv_lora_rank, self.qk_rope_head_dim], dim=-1)
        k_pe = k_pe.reshape(B, S, 1, self.qk_rope_head_dim)
        if reference:
            normed_kv = rmsnorm_ref(compressed, self.kv_a_layernorm.weight, self.eps)
        else:
            normed_kv = self.kv_a_layernorm(compressed.contiguous())
        return q_nope, q_pe, normed_kv, k_pe

    def _rope(self, q_pe, k_pe, rotary: RotaryPos):
        B, S = q_pe.shape[:2]
        cos, sin = rotary.gathered(B * S)
        cos, sin = cos.view(B, S, -1).to(q_pe.dtype), sin.view(B, S, -1).to(q_pe.dtype)
        return apply_rope_ref(interleaved_to_half(q_pe), cos, sin), apply_rope_ref(interleaved_to_half(k_pe), cos, sin)

    def forward(self, x, rotary: RotaryPos, cu_seqlens=None, reference: bool = False):
        B, S, _ = x.shape
        q_nope, q_pe, normed_kv, k_pe = self._project(x, reference)
        q_pe, k_pe = self._rope(q_pe, k_pe, rotary)
        if distributed.cp_size > 1 and not reference:
            from ..ops.ring_attention import mla_ring_attention_func

            o = mla_ring_attention_func(q_nope, q_pe, normed_kv.contiguous(), k_pe.contiguous(), self.kv_b_proj,
                                        sm_scale=self.softmax_scale, qk_nope_head_dim=self.qk_nope_head_dim,
                                        v_head_dim=self.v_head_dim)
        else:
            kvb = F.linear(normed_kv, self.kv_b_proj.weight) if reference else self.kv_b_proj(normed_kv)
            kv = kvb.view(B, S, self.num_heads, self.qk_nope_head_dim + self.v_head_dim)
            k_nope, v = torch.split(kv, [self.qk_nope_head_dim, self.v_head_dim], dim=-1)
            q = torch.cat([q_nope, q_pe], dim=-1)
            k = torch.cat([k_nope, k_pe.expand(-1, -1, self.num_heads, -1)], dim=-1)
            fn = attention_ref if reference else attention
            o = fn(q, k, v, causal=True, scale=self.softmax_scale, cu_seqlens=cu_seqlens)
        o = o.reshape(B, S, self.num_heads * self.v_head_dim)
        return F.linear(o, self.o_proj.weight) if reference else self.o_proj(o)


class DeepSeekV2DecoderLayer(nn.Module):
    def __init__(self, config: Any, layer_id: int):
        super().__init__()
        self.idx = layer_id
        H, eps = cfg_get(config, "hidden_size"), cfg_get(config, "rms_norm_eps", 1e-6)
        self.self_attn = DeepSeekV2Attention(config)
        has_experts = layer_id >= (cfg_get(config, "first_k_dense_replace", 0) or 0)
        self.mlp = DeepSeekV2MoE(config) if has_experts else DeepSeekV2MLP(config)
        self.input_layernorm = RMSNorm(H, eps=eps)
        self.post_attention_layernorm = RMSNorm(H, eps=eps)

    @property
    def is_moe(self) -> bool:
        return isinstance(self.mlp, DeepSeekV2MoE)

    def forward_stage1(self, hidden_states, rotary_posemb, cu_seqlens=None):
        x = self.input_layernorm(hidden_states)
        a = self.self_attn(x, rotary_posemb, cu_seqlens)
        x2, residual = self.post_attention_layernorm(a, residual=hidden_states)
        tokens = x2.view(-1, x2.shape[-1])
        if not self.is_moe:
            return tokens, residual, None
        if self.mlp.shared_experts is not None:
            residual = residual + self.mlp.shared_experts(tokens).view_as(residual)
        return tokens, residual, self.mlp.route(tokens)

    def forward_stage3(self, tokens, weights, routing):
        if not self.is_moe:
            return self.mlp(tokens)
        return self.mlp.experts_forward(tokens, weights, routing)

    def forward_stage5(self, outs, residual, routing):
        if self.is_moe:
            outs = self.mlp.finish(outs, routing)
        return residual + outs.view_as(residual)

    def reference_forward(self, hidden_states, rotary_posemb, cu_seqlens=None):
        eps = self.input_layernorm.eps
        h = hidden_states + self.self_attn(rmsnorm_ref(hidden_states, self.input_layernorm.weight, eps),
                                           rotary_posemb, cu_seqlens, reference=True)
        x2 = rmsnorm_ref(h, self.post_attention_layernorm.weight, eps)
        y = self.mlp.reference_forward(x2.view(-1, x2.shape[-1]))
        return h + y.view_as(h)


class DeepSeekV2Model(PipelineChunk):
    def build_layer(self, config, idx):
        return DeepSeekV2DecoderLayer(config, idx)

    def build_rotary(self, config):
        dim = cfg_get(config, "qk_rope_head_dim")
        base = rope_theta_of(config)
        rs = rope_scaling_of(config)
        inv_freq, attn_scale = None, 1.0
        if rs is not None and rs.get("rope_type", rs.get("type")) == "yarn":
            inv_freq = yarn_inv_freq(dim, base, rs["factor"], rs["original_max_position_embeddings"],
                                     rs.get("beta_fast", 32), rs.get("beta_slow", 1), truncate=True)
            attn_scale = float(yarn_mscale(rs["factor"], rs.get("mscale", 1.0)) /
                               yarn_mscale(rs["factor"], rs.get("mscale_all_dim", 0.0) or 0.0))
        dtype = torch.get_default_dtype()
        table_dtype = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
        return RotaryEmbedding(dim, cfg_get(config, "max_position_embeddings"), base, inv_freq=inv_freq,
                               attn_scale=attn_scale, table_dtype=table_dtype)
