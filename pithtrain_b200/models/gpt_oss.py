"""GPT-OSS (20B / 120B): GQA with biases, learned per-head attention sinks, alternating
sliding-window / full attention, top-k-then-softmax router with bias, experts with fused
interleaved gate/up weights, biases and the clamped SwiGLU.

Math specification: pithtrain/models/gpt_oss.py:29-92 (YaRN with ``truncate``), :95-157 (experts),
:160-190 (router), :218-269 (attention) of the reference. Unlike the reference (which raises for
``context_parallel_size > 1``, gpt_oss.py:361-362) the attention goes through the ring path when
the sequence is sharded: sinks enter the softmax denominator once at the final merge and
sliding-window layers fetch only the halo they can see.
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..contexts import distributed
from ..ops.attention import attention, attention_ref
from ..ops.common import grad_buffer
from ..ops.linear import FusedWeights, Linear, fused_linear
from ..ops.moe import ExpertWeights, moe_experts_ref
from ..ops.norm import RMSNorm, rmsnorm_ref
from ..ops.rope import apply_rope_ref, qk_norm_rope
from .common import (Gate, MoEBlock, PipelineChunk, RotaryEmbedding, RotaryPos, cfg_get, rope_scaling_of,
                     rope_theta_of, yarn_inv_freq)


class GptOssExperts(nn.Module):
    """Raw stacked parameters (checkpoint names carry no ``.weight`` suffix): ``gate_up_proj[E,2I,H]``
    with gate on even and up on odd rows, ``down_proj[E,H,I]`` and their biases."""

    def __init__(self, config: Any, num_experts: int):
        super().__init__()
        H, I = cfg_get(config, "hidden_size"), cfg_get(config, "intermediate_size")
        self.num_experts = num_experts
        self.swiglu_limit = float(cfg_get(config, "swiglu_limit", 7.0))
        self.alpha = 1.702
        self.gate_up_proj = nn.Parameter(torch.empty(num_experts, 2 * I, H))
        self.gate_up_proj_bias = nn.Parameter(torch.zeros(num_experts, 2 * I))
        self.down_proj = nn.Parameter(torch.empty(num_experts, H, I))
        self.down_proj_bias = nn.Parameter(torch.zeros(num_experts, H))
        nn.init.normal_(self.gate_up_proj, std=0.02)
        nn.init.normal_(self.down_proj, std=0.02)
        self._wq_cache = None

    def expert_weights(self) -> ExpertWeights:
        return ExpertWeights(self.gate_up_proj, self.down_proj, lambda: grad_buffer(self.gate_up_proj),
                             lambda: grad_buffer(self.down_proj), b1=self.gate_up_proj_bias, b2=self.down_proj_bias,
                             interleaved=True, alpha=self.alpha, limit=self.swiglu_limit)

    def reference(self, x, w, eids):
        return moe_experts_ref(x, w, eids, self.gate_up_proj, self.down_proj, self.gate_up_proj_bias,
                               self.down_proj_bias, interleaved=True, alpha=self.alpha, limit=self.swiglu_limit)


class GptOssTopKRouter(Gate):
    def __init__(self, config: Any):
        super().__init__(cfg_get(config, "hidden_size"), cfg_get(config, "num_local_experts"),
                         cfg_get(config, "num_experts_per_tok"), mode="topk_softmax", bias=True)


class GptOssMoE(MoEBlock):
    def __init__(self, config: Any):
        E, k = cfg_get(config, "num_local_experts"), cfg_get(config, "num_experts_per_tok")
        # the checkpoint name of the gate is ``router``
        super().__init__(GptOssTopKRouter(config), GptOssExperts(config, E // distributed.ep_size), E, k,
                         gate_attr="router")
        self.hidden_size = cfg_get(config, "hidden_size")


class GptOssAttention(nn.Module):
    def __init__(self, config: Any, is_sliding: bool):
        super().__init__()
        H = cfg_get(config, "hidden_size")
        self.num_heads = cfg_get(config, "num_attention_heads")
        self.num_kv_heads = cfg_get(config, "num_key_value_heads")
        self.head_dim = cfg_get(config, "head_dim")
        self.scaling = self.head_dim ** -0.5
        self.is_sliding = is_sliding
        self.sliding_window = cfg_get(config, "sliding_window")
        bias = bool(cfg_get(config, "attention_bias", True))
        self.q_proj = Linear(H, self.num_heads * self.head_dim, bias=bias)
        self.k_proj = Linear(H, self.num_kv_heads * self.head_dim, bias=bias)
        self.v_proj = Linear(H, self.num_kv_heads * self.head_dim, bias=bias)
        self.o_proj = Linear(self.num_heads * self.head_dim, H, bias=bias)
        self.sinks = nn.Parameter(torch.zeros(self.num_heads))
        self.fused_qkv = FusedWeights([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], layout="rows")

    @property
    def window_left(self) -> Optional[int]:
        return self.sliding_window - 1 if self.is_sliding else None

    def forward(self, x, rotary: RotaryPos, cu_seqlens=None):
        B, S, H = x.shape
        n = B * S
        biases = [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias] if self.q_proj.bias is not None else None
        qkv = fused_linear(x.view(n, H), self.fused_qkv, biases)
        q, k, v = qk_norm_rope(qkv, None, None, rotary.cos, rotary.sin, self.num_heads, self.num_kv_heads,
                               self.head_dim, positions=rotary.token_positions(n), S=S)
        q = q.view(B, S, self.num_heads, self.head_dim)
        k = k.view(B, S, self.num_kv_heads, self.head_dim)
        v = v.reshape(B, S, self.num_kv_heads, self.head_dim)
        sinks = self.sinks
        if distributed.cp_size > 1:
            from ..ops.ring_attention import ring_attention_func

            o = ring_attention_func(q, k, v, softmax_scale=self.scaling, window_left=self.window_left, sinks=sinks)
        else:
            o = attention(q, k, v, causal=True, scale=self.scaling, window_left=self.window_left, sinks=sinks,
                          cu_seqlens=cu_seqlens)
        return self.o_proj(o.reshape(B, S, self.num_heads * self.head_dim))

    def reference(self, x, rotary: RotaryPos, cu_seqlens=None):
        B, S, _ = x.shape
        q = F.linear(x, self.q_proj.weight, self.q_proj.bias).view(B, S, self.num_heads, self.head_dim)
        k = F.linear(x, self.k_proj.weight, self.k_proj.bias).view(B, S, self.num_kv_heads, self.head_dim)
        v = F.linear(x, self.v_proj.weight, self.v_proj.bias).view(B, S, self.num_kv_heads, self.head_dim)
        cos, sin = rotary.gathered(B * S)
        cos, sin = cos.view(B, S, -1).to(q.dtype), sin.view(B, S, -1).to(q.dtype)
        q, k = apply_rope_ref(q, cos, sin), apply_rope_ref(k, cos, sin)
        o = attention_ref(q, k, v, causal=True, scale=self.scaling, window_left=self.window_left, sinks=self.sinks,
                          cu_seqlens=cu_seqlens)
        return F.linear(o.reshape(B, S, -1), self.o_proj.weight, self.o_proj.bias)


class GptOssDecoderLayer(nn.Module):
    def __init__(self, config: Any, layer_idx: int):
        super().__init__()
        self.idx = layer_idx
        H, eps = cfg_get(config, "hidden_size"), cfg_get(config, "rms_norm_eps", 1e-5)
        layer_types = cfg_get(config, "layer_types")
        if layer_types is None:
            layer_types = ["sliding_attention" if i % 2 == 0 else "full_attention"
                           for i in range(cfg_get(config, "num_hidden_layers"))]
        self.self_attn = GptOssAttention(config, layer_types[layer_idx] == "sliding_attention")
        self.mlp = GptOssMoE(config)
        self.input_layernorm = RMSNorm(H, eps=eps)
        self.post_attention_layernorm = RMSNorm(H, eps=eps)

    def forward_stage1(self, hidden_states, rotary_posemb, cu_seqlens=None):
        x = self.input_layernorm(hidden_states)
        a = self.self_attn(x, rotary_posemb, cu_seqlens)
        x2, residual = self.post_attention_layernorm(a, residual=hidden_states)
        tokens = x2.view(-1, x2.shape[-1])
        return tokens, residual, self.mlp.route(tokens)

    def forward_stage3(self, tokens, weights, routing):
        return self.mlp.experts_forward(tokens, weights, routing)

    def forward_stage5(self, outs, residual, routing):
        return residual + self.mlp.finish(outs, routing).view_as(residual)

    def reference_forward(self, hidden_states, rotary_posemb, cu_seqlens=None):
        eps = self.input_layernorm.eps
        h = hidden_states + self.self_attn.reference(rmsnorm_ref(hidden_states, self.input_layernorm.weight, eps),
                                                     rotary_posemb, cu_seqlens)
        x2 = rmsnorm_ref(h, self.post_attention_layernorm.weight, eps)
        return h + self.mlp.reference_forward(x2.view(-1, x2.shape[-1])).view_as(h)


class GptOssModel(PipelineChunk):
    def build_layer(self, config, idx):
        return GptOssDecoderLayer(config, idx)

    def build_norm(self, config):
        return RMSNorm(cfg_get(config, "hidden_size"), eps=cfg_get(config, "rms_norm_eps", 1e-5))

    def build_rotary(self, config):
        dim, base = cfg_get(config, "head_dim"), rope_theta_of(config)
        rs = rope_scaling_of(config)
        inv_freq, attn_scale = None, 1.0
        if rs is not None and rs.get("rope_type", rs.get("type")) == "yarn":
            ctx = cfg_get(config, "initial_context_length") or rs.get("original_max_position_embeddings", 4096)
            inv_freq = yarn_inv_freq(dim, base, rs["factor"], ctx, rs.get("beta_fast", 32), rs.get("beta_slow", 1),
                                     truncate=bool(rs.get("truncate", True)))
            attn_scale = 0.1 * math.log(rs["factor"]) + 1.0
        dtype = torch.get_default_dtype()
        table_dtype = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
        return RotaryEmbedding(dim, cfg_get(config, "max_position_embeddings"), base, inv_freq=inv_freq,
                               attn_scale=attn_scale, table_dtype=table_dtype)
