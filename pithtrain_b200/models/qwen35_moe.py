"""Qwen3.5-MoE (text): three Gated-DeltaNet linear-attention layers per gated full-attention layer,
zero-centred RMSNorm, partial rotary embedding, fused gate/up experts and a sigmoid-gated shared
expert.

Math specification: pithtrain/models/qwen35_moe.py:24-47 (norms), :67-113 (Gated DeltaNet),
:116-163 (gated attention), :179-247 (MoE block) of the reference. Like the reference this family
supports neither context parallelism nor packed sequences.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..contexts import distributed
from ..ops.attention import attention, attention_ref
from ..ops.common import grad_buffer
from ..ops.gated_delta_rule import gated_delta_rule, gated_delta_rule_recurrent
from ..ops.linear import FusedWeights, Linear, fused_linear
from ..ops.moe import ExpertWeights, moe_experts_ref
from ..ops.norm import RMSNorm, rmsnorm_ref
from ..ops.rope import apply_rope_ref
from .common import DenseMLP, Gate, MoEBlock, PipelineChunk, RotaryEmbedding, RotaryPos, cfg_get, rope_theta_of


class Qwen35MoeRMSNormGated(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.weight._init_fill = 1.0
        self.eps = eps

    def forward(self, x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (out * self.weight.float() * F.silu(gate.float())).type_as(x)


class Qwen35MoeGatedDeltaNet(nn.Module):
    def __init__(self, config: Any, layer_idx: int):
        super().__init__()
        H = cfg_get(config, "hidden_size")
        self.num_k_heads, self.num_v_heads = cfg_get(config, "linear_num_key_heads"), cfg_get(config, "linear_num_value_heads")
        self.head_k_dim, self.head_v_dim = cfg_get(config, "linear_key_head_dim"), cfg_get(config, "linear_value_head_dim")
        self.key_dim, self.value_dim = self.head_k_dim * self.num_k_heads, self.head_v_dim * self.num_v_heads
        self.conv_kernel_size = cfg_get(config, "linear_conv_kernel_dim")
        self.conv_dim = self.key_dim * 2 + self.value_dim
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, bias=False, kernel_size=self.conv_kernel_size,
                                groups=self.conv_dim, padding=self.conv_kernel_size - 1)
        self.dt_bias = nn.Parameter(torch.ones(self.num_v_heads))
        self.dt_bias._init_fill = 1.0
        self.A_log = nn.Parameter(torch.zeros(self.num_v_heads))
        self.A_log._init_fn = lambda p: p.copy_(torch.log(torch.empty(p.shape, dtype=torch.float32).uniform_(1e-3, 16)).to(p.dtype))
        if not self.A_log.is_meta:
            with torch.no_grad():
                self.A_log._init_fn(self.A_log)
        self.norm = Qwen35MoeRMSNormGated(self.head_v_dim, eps=cfg_get(config, "rms_norm_eps", 1e-6))
        self.in_proj_qkv = Linear(H, self.key_dim * 2 + self.value_dim, bias=False)
        self.in_proj_z = Linear(H, self.value_dim, bias=False)
        self.in_proj_b = Linear(H, self.num_v_heads, bias=False)
        self.in_proj_a = Linear(H, self.num_v_heads, bias=False)
        self.out_proj = Linear(self.value_dim, H, bias=False)

    def forward(self, x: torch.Tensor, reference: bool = False) -> torch.Tensor:
        B, S, _ = x.shape
        lin = (lambda m, t: F.linear(t, m.weight)) if reference else (lambda m, t: m(t))
        mixed = lin(self.in_proj_qkv, x).transpose(1, 2)
        z = lin(self.in_proj_z, x).reshape(B, S, -1, self.head_v_dim)
        b, a = lin(self.in_proj_b, x), lin(self.in_proj_a, x)
        mixed = F.silu(self.conv1d(mixed)[..., :S]).transpose(1, 2)
        q, k, v = torch.split(mixed, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q = F.normalize(q.reshape(B, S, -1, self.head_k_dim), dim=-1)
        k = F.normalize(k.reshape(B, S, -1, self.head_k_dim), dim=-1)
        v = v.reshape(B, S, -1, self.head_v_dim)
        beta = b.sigmoid()
        g = -self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias.float())
        rep = self.num_v_heads // self.num_k_heads
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
        fn = gated_delta_rule_recurrent if reference else gated_delta_rule
        o = fn(q, k, v, g, beta).reshape(-1, self.head_v_dim)
        o = self.norm(o, z.reshape(-1, self.head_v_dim)).reshape(B, S, -1)
        return lin(self.out_proj, o)


class Qwen35MoeAttention(nn.Module):
    """Full attention whose q projection also emits a per-head output gate."""

    def __init__(self, config: Any):
        super().__init__()
        H = cfg_get(config, "hidden_size")
        self.num_heads, self.num_kv_heads = cfg_get(config, "num_attention_heads"), cfg_get(config, "num_key_value_heads")
        self.head_dim = cfg_get(config, "head_dim")
        self.scaling = self.head_dim ** -0.5
        self.eps = cfg_get(config, "rms_norm_eps", 1e-6)
        bias = bool(cfg_get(config, "attention_bias", False))
        self.q_proj = Linear(H, self.num_heads * self.head_dim * 2, bias=bias)
        self.k_proj = Linear(H, self.num_kv_heads * self.head_dim, bias=bias)
        self.v_proj = Linear(H, self.num_kv_heads * self.head_dim, bias=bias)
        self.o_proj = Linear(self.num_heads * self.head_dim, H, bias=bias)
        self.q_norm = RMSNorm(self.head_dim, eps=self.eps, zero_centered=True)
        self.k_norm = RMSNorm(self.head_dim, eps=self.eps, zero_centered=True)
        self.fused_qkv = FusedWeights([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], layout="rows")

    @staticmethod
    def partial_rope(x, cos, sin):
        rd = cos.shape[-1]
        return torch.cat([apply_rope_ref(x[..., :rd], cos, sin), x[..., rd:]], dim=-1)

    def forward(self, x, rotary: RotaryPos, reference: bool = False):
        B, S, H = x.shape
        nq = self.num_heads * self.head_dim * 2
        nkv = self.num_kv_heads * self.head_dim
        if reference:
            qg = F.linear(x, self.q_proj.weight, self.q_proj.bias)
            kx = F.linear(x, self.k_proj.weight, self.k_proj.bias)
            vx = F.linear(x, self.v_proj.weight, self.v_proj.bias)
        else:
            biases = [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias] if self.q_proj.bias is not None else None
            qkv = fused_linear(x.view(B * S, H), self.fused_qkv, biases).view(B, S, -1)
            qg, kx, vx = qkv[..., :nq], qkv[..., nq:nq + nkv], qkv[..., nq + nkv:]
        q, gate = torch.chunk(qg.reshape(B, S, self.num_heads, self.head_dim * 2), 2, dim=-1)
        gate = gate.reshape(B, S, -1)
        k = kx.reshape(B, S, self.num_kv_heads, self.head_dim)
        v = vx.reshape(B, S, self.num_kv_heads, self.head_dim)
        if reference:
            q = rmsnorm_ref(q, self.q_norm.weight, self.eps, zero_centered=True)
            k = rmsnorm_ref(k, self.k_norm.weight, self.eps, zero_centered=True)
        else:
            q, k = self.q_norm(q.contiguous()), self.k_norm(k.contiguous())
        cos, sin = rotary.gathered(B * S)
        cos, sin = cos.view(B, S, -1).to(q.dtype), sin.view(B, S, -1).to(q.dtype)
        q, k = self.partial_rope(q, cos, sin), self.partial_rope(k, cos, sin)
        o = (attention_ref if reference else attention)(q, k, v, causal=True, scale=self.scaling)
        o = o.reshape(B, S, -1) * torch.sigmoid(gate)
        return F.linear(o, self.o_proj.weight, self.o_proj.bias) if reference else self.o_proj(o)


class _FusedExpertProj(nn.Module):
    def __init__(self, num_experts: int, in_features: int, out_features: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        nn.init.normal_(self.weight, std=0.02)


class Qwen35MoeExperts(nn.Module):
    """Fused ``gate_up_proj.weight [E, 2I, H]`` (gate rows first) and ``down_proj.weight [E, H, I]``."""

    def __init__(self, config: Any, num_experts: int):
        super().__init__()
        H, I = cfg_get(config, "hidden_size"), cfg_get(config, "moe_intermediate_size")
        self.num_experts, self.hidden_size, self.moe_intermediate_size = num_experts, H, I
        self.gate_up_proj = _FusedExpertProj(num_experts, H, 2 * I)
        self.down_proj = _FusedExpertProj(num_experts, I, H)

    def expert_weights(self) -> ExpertWeights:
        return ExpertWeights(self.gate_up_proj.weight, self.down_proj.weight, lambda: grad_buffer(self.gate_up_proj.weight),
                             lambda: grad_buffer(self.down_proj.weight))

    def reference(self, x, w, eids):
        return moe_experts_ref(x, w, eids, self.gate_up_proj.weight, self.down_proj.weight)


class Qwen35MoeSparseMoeBlock(MoEBlock):
    def __init__(self, config: Any):
        E, k, H = cfg_get(config, "num_experts"), cfg_get(config, "num_experts_per_tok"), cfg_get(config, "hidden_size")
        gate = Gate(H, E, k, mode="softmax_topk", norm_topk_prob=True)
        super().__init__(gate, Qwen35MoeExperts(config, E // distributed.ep_size), E, k)
        self.hidden_size = H
        self.shared_expert = DenseMLP(H, cfg_get(config, "shared_expert_intermediate_size"))
        self.shared_expert_gate = Linear(H, 1, bias=False)

    def shared_out(self, tokens: torch.Tensor, reference: bool = False) -> torch.Tensor:
        if reference:
            return torch.sigmoid(F.linear(tokens, self.shared_expert_gate.weight)) * self.shared_expert.reference(tokens)
        return torch.sigmoid(F.linear(tokens, self.shared_expert_gate.weight)) * self.shared_expert(tokens)

    def reference_forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return super().reference_forward(tokens) + self.shared_out(tokens, reference=True)


class Qwen35MoeDecoderLayer(nn.Module):
    def __init__(self, config: Any, layer_idx: int):
        super().__init__()
        self.idx = layer_idx
        H, eps = cfg_get(config, "hidden_size"), cfg_get(config, "rms_norm_eps", 1e-6)
        layer_types = cfg_get(config, "layer_types")
        if layer_types is None:
            interval = cfg_get(config, "full_attention_interval", 4)
            layer_types = ["full_attention" if (i + 1) % interval == 0 else "linear_attention"
                           for i in range(cfg_get(config, "num_hidden_layers"))]
        self.layer_type = layer_types[layer_idx]
        self.is_linear = self.layer_type == "linear_attention"
        if self.is_linear:
            self.linear_attn = Qwen35MoeGatedDeltaNet(config, layer_idx)
        else:
            self.self_attn = Qwen35MoeAttention(config)
        self.mlp = Qwen35MoeSparseMoeBlock(config)
        self.input_layernorm = RMSNorm(H, eps=eps, zero_centered=True)
        self.post_attention_layernorm = RMSNorm(H, eps=eps, zero_centered=True)

    def _mixer(self, x, rotary, reference=False):
        if self.is_linear:
            return self.linear_attn(x, reference=reference)
        return self.self_attn(x, rotary, reference=reference)

    def forward_stage1(self, hidden_states, rotary_posemb, cu_seqlens=None):
        assert cu_seqlens is None, "packed sequences are not implemented for Gated DeltaNet"
        x = self.input_layernorm(hidden_states)
        a = self._mixer(x, rotary_posemb)
        x2, residual = self.post_attention_layernorm(a, residual=hidden_states)
        tokens = x2.view(-1, x2.shape[-1])
        residual = residual + self.mlp.shared_out(tokens).view_as(residual)
        return tokens, residual, self.mlp.route(tokens)

    def forward_stage3(self, tokens, weights, routing):
        return self.mlp.experts_forward(tokens, weights, routing)

    def forward_stage5(self, outs, residual, routing):
        return residual + self.mlp.finish(outs, routing).view_as(residual)

    def reference_forward(self, hidden_states, rotary_posemb, cu_seqlens=None):
        eps = self.input_layernorm.eps
        h = hidden_states + self._mixer(rmsnorm_ref(hidden_states, self.input_layernorm.weight, eps, zero_centered=True),
                                        rotary_posemb, reference=True)
        x2 = rmsnorm_ref(h, self.post_attention_layernorm.weight, eps, zero_centered=True)
        return h + self.mlp.reference_forward(x2.view(-1, x2.shape[-1])).view_as(h)


class Qwen35MoeModel(PipelineChunk):
    supports_cp = False
    supports_packed = False

    def __init__(self, config: Any, phase: int):
        if distributed.cp_size > 1:
            raise NotImplementedError("Qwen35MoeModel doesn't support context parallelism.")
        super().__init__(config, phase)

    def build_layer(self, config, idx):
        return Qwen35MoeDecoderLayer(config, idx)

    def build_norm(self, config):
        return RMSNorm(cfg_get(config, "hidden_size"), eps=cfg_get(config, "rms_norm_eps", 1e-6), zero_centered=True)

    def build_rotary(self, config):
        rp = cfg_get(config, "rope_parameters") or {}
        factor = rp.get("partial_rotary_factor", cfg_get(config, "partial_rotary_factor", 1.0))
        rotary_dim = int(cfg_get(config, "head_dim") * factor)
        dtype = torch.get_default_dtype()
        table_dtype = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
        return RotaryEmbedding(rotary_dim, cfg_get(config, "max_position_embeddings"), rope_theta_of(config),
                               table_dtype=table_dtype)
