"""Parameter and FLOP counts derived from a model config (used for MFU and the memory estimator)."""

from __future__ import annotations

from typing import Any, Tuple


def _g(c: Any, k: str, d=None):
    return c.get(k, d) if isinstance(c, dict) else getattr(c, k, d)


def attention_dims(config: Any) -> Tuple[int, int, int]:
    """(query heads, qk head dim, v head dim)."""
    hq = _g(config, "num_attention_heads")
    if _g(config, "model_type") == "deepseek_v2":
        return hq, _g(config, "qk_nope_head_dim") + _g(config, "qk_rope_head_dim"), _g(config, "v_head_dim")
    d = _g(config, "head_dim") or _g(config, "hidden_size") // hq
    return hq, d, d


def attention_params(config: Any) -> int:
    H = _g(config, "hidden_size")
    hq, dqk, dv = attention_dims(config)
    if _g(config, "model_type") == "deepseek_v2":
        r, rope = _g(config, "kv_lora_rank"), _g(config, "qk_rope_head_dim")
        nope = _g(config, "qk_nope_head_dim")
        q_lora = _g(config, "q_lora_rank")
        q = H * hq * dqk if not q_lora else H * q_lora + q_lora * hq * dqk
        return q + H * (r + rope) + r * hq * (nope + dv) + hq * dv * H
    hkv = _g(config, "num_key_value_heads", hq)
    return H * hq * dqk + 2 * H * hkv * dqk + hq * dv * H


def moe_layer_counts(config: Any) -> Tuple[int, int]:
    """(number of MoE layers, number of dense-MLP layers)."""
    L = _g(config, "num_hidden_layers")
    dense = _g(config, "first_k_dense_replace", 0) or 0
    return L - dense, dense


def expert_count(config: Any) -> Tuple[int, int, int]:
    """(routed experts, top-k, shared experts)."""
    E = _g(config, "num_experts") or _g(config, "n_routed_experts") or _g(config, "num_local_experts")
    k = _g(config, "num_experts_per_tok")
    shared = _g(config, "n_shared_experts", 0) or (1 if _g(config, "shared_expert_intermediate_size") else 0)
    return E, k, shared


def expert_ffn_params(config: Any) -> int:
    H = _g(config, "hidden_size")
    I = _g(config, "moe_intermediate_size") or _g(config, "intermediate_size")
    return 3 * H * I


def active_matmul_params(config: Any) -> int:
    """Matmul parameters touched per token (lm_head included, embedding lookup excluded)."""
    H, V = _g(config, "hidden_size"), _g(config, "vocab_size")
    moe_layers, dense_layers = moe_layer_counts(config)
    E, k, shared = expert_count(config)
    per_moe = attention_params(config) + H * E + (k + shared) * expert_ffn_params(config)
    if _g(config, "shared_expert_intermediate_size"):
        per_moe += 3 * H * _g(config, "shared_expert_intermediate_size") - shared * expert_ffn_params(config)
    per_dense = attention_params(config) + 3 * H * (_g(config, "intermediate_size") or 0)
    return moe_layers * per_moe + dense_layers * per_dense + H * V


def total_params(config: Any) -> int:
    H, V = _g(config, "hidden_size"), _g(config, "vocab_size")
    moe_layers, dense_layers = moe_layer_counts(config)
    E, k, shared = expert_count(config)
    per_moe = attention_params(config) + H * E + (E + shared) * expert_ffn_params(config) + 2 * H
    per_dense = attention_params(config) + 3 * H * (_g(config, "intermediate_size") or 0) + 2 * H
    return moe_layers * per_moe + dense_layers * per_dense + 2 * H * V + H
