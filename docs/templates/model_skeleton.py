"""Skeleton of a model family for pithtrain_b200 (copy into pithtrain_b200/models/<name>.py and fill in)."""

from __future__ import annotations

from typing import Any, Optional

import torch
import torch.nn as nn

from pithtrain_b200.models.common import Gate, MoEBlock, PipelineChunk, RotaryEmbedding, SwiGLUExperts, cfg_get, rope_theta_of
from pithtrain_b200.contexts import distributed
from pithtrain_b200.ops.norm import RMSNorm, rmsnorm_ref


class MyAttention(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        # projections (ops.linear.Linear), FusedWeights([...], layout="rows") for q/k/v, norms

    def forward(self, x: torch.Tensor, rotary, cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError  # fused_linear -> qk_norm_rope -> attention / ring_attention_func -> o_proj

    def reference(self, x: torch.Tensor, rotary, cu_seqlens=None) -> torch.Tensor:
        raise NotImplementedError  # same math with torch.nn.functional ops and ops.attention.attention_ref


class MyMoE(MoEBlock):
    def __init__(self, config: Any):
        E, k = cfg_get(config, "num_experts"), cfg_get(config, "num_experts_per_tok")
        H, I = cfg_get(config, "hidden_size"), cfg_get(config, "moe_intermediate_size")
        gate = Gate(H, E, k, mode="softmax_topk")
        super().__init__(gate, SwiGLUExperts(E // distributed.ep_size, H, I), E, k)


class MyDecoderLayer(nn.Module):
    def __init__(self, config: Any, idx: int):
        super().__init__()
        self.idx = idx
        H, eps = cfg_get(config, "hidden_size"), cfg_get(config, "rms_norm_eps", 1e-6)
        self.self_attn, self.mlp = MyAttention(config), MyMoE(config)
        self.input_layernorm, self.post_attention_layernorm = RMSNorm(H, eps=eps), RMSNorm(H, eps=eps)

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
        h = hidden_states + self.self_attn.reference(rmsnorm_ref(hidden_states, self.input_layernorm.weight, eps), rotary_posemb, cu_seqlens)
        x2 = rmsnorm_ref(h, self.post_attention_layernorm.weight, eps)
        return h + self.mlp.reference_forward(x2.view(-1, x2.shape[-1])).view_as(h)


class MyModel(PipelineChunk):
    """``MyModel(config, phase)``: phase 0/1 = this rank's two pipeline chunks, -1 = the whole model."""

    def build_layer(self, config, idx):
        return MyDecoderLayer(config, idx)

    def build_rotary(self, config):
        dim = cfg_get(config, "head_dim") or cfg_get(config, "hidden_size") // cfg_get(config, "num_attention_heads")
        return RotaryEmbedding(dim, cfg_get(config, "max_position_embeddings"), rope_theta_of(config))
