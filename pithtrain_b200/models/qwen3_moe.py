"""Qwen3-MoE (Qwen3-30B-A3B, Qwen3-235B-A22B): GQA attention with per-head QK RMSNorm and
rotate-half RoPE, softmax-then-top-k router, SwiGLU experts.

Math specification: pithtrain/models/qwen3_moe.py:68-120,123-176,247-261 of the reference. The
attention block runs as: fused q/k/v GEMM -> fused QK-norm + RoPE kernel -> attention -> o_proj;
``reference_forward`` restates the same math with plain PyTorch ops and is the oracle for the
engine tests.
"""

from __future__ import annotations

from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..contexts import distributed
from ..ops.attention import attention, attention_ref
from ..ops.linear import FusedWeights, Linear, fused_linear
from ..ops.norm import RMSNorm, rmsnorm_ref
from ..ops.rope import apply_rope_ref, qk_norm_rope
from .common import (Gate, MoEBlock, PipelineChunk, RotaryEmbedding, RotaryPos, SwiGLUExperts, cfg_get,
                     rope_theta_of)


class Qwen3MoeAttention(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        H = cfg_get(config, "hidden_size")
        self.num_heads = cfg_get(config, "num_attention_heads")
        self.num_kv_heads = cfg_get(config, "num_key_value_heads")
        self.head_dim = cfg_get(config, "head_dim") or H // self.num_heads
        self.scaling = self.head_dim ** -0.5
        self.eps = cfg_get(config, "rms_norm_eps", 1e-6)
        bias = bool(cfg_get(config, "attention_bias", False))
        self.q_proj = Linear(H, self.num_heads * self.head_dim, bias=bias)
        self.k_proj = Linear(H, self.num_kv_heads * self.head_dim, bias=bias)
        self.v_proj = Linear(H, self.num_kv_heads * self.head_dim, bias=bias)
        self.o_proj = Linear(self.num_heads * self.head_dim, H, bias=bias)
        self.q_norm = RMSNorm(self.head_dim, eps=self.eps)
        self.k_norm = RMSNorm(self.head_dim, eps=self.eps)
        self.fused_qkv = FusedWeights([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], layout="rows")

    def forward(self, x: torch.Tensor, rotary: RotaryPos, cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S, H = x.shape
        n = B * S
        biases = [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias] if self.q_proj.bias is not None else None
        qkv = fused_linear(x.view(n, H), self.fused_qkv, biases)
        q, k, v = qk_norm_rope(qkv, self.q_norm.weight, self.k_norm.weight, rotary.cos, rotary.sin,
                               self.num_heads, self.num_kv_heads, self.head_dim, self.eps,
                               positions=rotary.token_positions(n), S=S)
        q = q.view(B, S, self.num_heads, self.head_dim)
        k = k.view(B, S, self.num_kv_heads, self.head_dim)
        v = v.reshape(B, S, self.num_kv_heads, self.head_dim)
        if distributed.cp_size > 1:
            from ..ops.ring_attention import ring_attention_func

            o = ring_attention_func(q, k, v, softmax_scale=self.scaling)
        else:
            o = attention(q, k, v, causal=True, scale=self.scaling, cu_seqlens=cu_seqlens)
        return self.o_proj(o.reshape(B, S, self.num_heads * self.head_dim))

    def reference(self, x: torch.Tensor, rotary: RotaryPos, cu_seqlens=None) -> torch.Tensor:
        B, S, H = x.shape
        n = B * S
        q = self.q_proj.weight, self.k_proj.weight
        qh = F.linear(x, self.q_proj.weight, self.q_proj.bias).view(B, S, self.num_heads, self.head_dim)
        kh = F.linear(x, self.k_proj.weight, self.k_proj.bias).view(B, S, self.num_kv_heads, self.head_dim)
        vh = F.linear(x, self.v_proj.weight, self.v_proj.bias).view(B, S, self.num_kv_heads, self.head_dim)
        qh = rmsnorm_ref(qh, self.q_norm.weight, self.eps)
        kh = rmsnorm_ref(kh, self.k_norm.weight, self.eps)
        cos, sin = rotary.gathered(n)
        cos, sin = cos.view(B, S, -1).to(qh.dtype), sin.view(B, S, -1).to(qh.dtype)
        qh, kh = apply_rope_ref(qh, cos, sin), apply_rope_ref(kh, cos, sin)
        o = attention_ref(qh, kh, vh, causal=True, scale=self.scaling, cu_seqlens=cu_seqlens)
        return F.linear(o.reshape(B, S, -1), self.o_proj.weight, self.o_proj.bias)


class Qwen3MoeMoE(MoEBlock):
    def __init__(self, config: Any):
        E, k = cfg_get(config, "num_experts"), cfg_get(config, "num_experts_per_tok")
        H, I = cfg_get(config, "hidden_size"), cfg_get(config, "moe_intermediate_size")
        epr = E // distributed.ep_size
        gate = Gate(H, E, k, mode="softmax_topk", norm_topk_prob=bool(cfg_get(config, "norm_topk_prob", False)))
        super().__init__(gate, SwiGLUExperts(epr, H, I), E, k)


class Qwen3MoeDecoderLayer(nn.Module):
    def __init__(self, config: Any, idx: int):
        super().__init__()
        self.idx = idx
        H, eps = cfg_get(config, "hidden_size"), cfg_get(config, "rms_norm_eps", 1e-6)
        self.self_attn = Qwen3MoeAttention(config)
        self.mlp = Qwen3MoeMoE(config)
        self.input_layernorm = RMSNorm(H, eps=eps)
        self.post_attention_layernorm = RMSNorm(H, eps=eps)

    def forward_stage1(self, hidden_states, rotary_posemb, cu_seqlens=None):
        x = self.input_layernorm(hidden_states)
        a = self.self_attn(x, rotary_posemb, cu_seqlens)
        x2, residual = self.post_attention_layernorm(a, residual=hidden_states)
        tokens = x2.view(-1, x2.shape[-1])
        routing = self.mlp.route(tokens)
        return tokens, residual, routing

    def forward_stage3(self, tokens, weights, routing):
        return self.mlp.experts_forward(tokens, weights, routing)

    def forward_stage5(self, outs, residual, routing):
        y = self.mlp.finish(outs, routing)
        return residual + y.view_as(residual)

    def reference_forward(self, hidden_states, rotary_posemb, cu_seqlens=None):
        eps = self.input_layernorm.eps
        h = hidden_states + self.self_attn.reference(rmsnorm_ref(hidden_states, self.input_layernorm.weight, eps),
                                                     rotary_posemb, cu_seqlens)
        x2 = rmsnorm_ref(h, self.post_attention_layernorm.weight, eps)
        y = self.mlp.reference_forward(x2.view(-1, x2.shape[-1]))
        return h + y.view_as(h)


class Qwen3MoeModel(PipelineChunk):
    """``Qwen3MoeModel(config, phase)``: phase 0/1 = the rank's two pipeline chunks, -1 = whole model."""

    def build_layer(self, config, idx):
        return Qwen3MoeDecoderLayer(config, idx)

    def build_rotary(self, config):
        H = cfg_get(config, "hidden_size")
        dim = cfg_get(config, "head_dim") or H // cfg_get(config, "num_attention_heads")
        dtype = torch.get_default_dtype()
        table_dtype = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
        return RotaryEmbedding(dim, cfg_get(config, "max_position_embeddings"), rope_theta_of(config),
                               table_dtype=table_dtype)
