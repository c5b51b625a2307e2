"""Static memory of one rank: parameters, gradient accumulators, optimizer state.

The numbers follow this framework's own layout (pithtrain_b200/parallel/flat_shard.py): every rank keeps
the full flat parameter and gradient buffers of its two pipeline chunks (experts: only its
``E / ep`` local experts); optimizer state exists only for the parameters a rank owns, i.e. it is
divided by the size of the shard group (dp×cp for experts, dp×cp×ep for the rest), and can live in
pinned host memory instead of HBM. The reference's estimator models FSDP2 shards plus gathered
copies instead (tools/memory_estimator/model_profile.py of the reference).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

from ...dualpipe.dualpipev import layer_partition

DTYPE_BYTES = {"bf16": 2, "fp32": 4, "fp16": 2}


@dataclass
class ParallelCfg:
    pp: int = 1
    ep: int = 1
    cp: int = 1
    dp: int = 1
    micro_batch_size: int = 1
    global_batch_size: int = 32
    sequence_length: int = 4096
    grad_dtype: str = "bf16"
    optimizer: str = "muon"  # "muon" (momentum; AdamW for non-matrix params) or "adamw"
    momentum_dtype: str = "bf16"
    offload_optimizer_state: bool = False
    resident_state_gb: float = 0.0  # with offload: GiB of optimizer state kept on the device anyway
    ep_backend: str = "fused"  # "fused" (symmetric buffers) or "nccl"
    fp8_training: bool = False  # block-scaled e4m3 forward / input-gradient GEMMs: cached quantised weight copies
    capacity_factor: Optional[float] = None
    reshard_params: bool = False  # DistributedCfg.reshard_params: owned parameters in a buffer of their own

    @property
    def world(self) -> int:
        return self.pp * self.ep * self.cp * self.dp

    @property
    def num_chunks(self) -> int:
        return max(1, self.global_batch_size // (self.micro_batch_size * self.dp * self.ep))

    @property
    def tokens_per_microbatch(self) -> int:
        return self.micro_batch_size * self.sequence_length // self.cp


@dataclass
class LayerShape:
    """Per-layer parameter counts (elements) and the dimensions the activation model needs."""

    kind: str  # "moe" or "dense"
    attn_kind: str  # "gqa", "mla", "linear" (gated delta net), "gated_gqa"
    attn_params: int
    expert_params_per_expert: int
    dense_mlp_params: int
    shared_params: int
    router_params: int
    norm_params: int


@dataclass
class ModelDims:
    model_type: str
    H: int
    L: int
    V: int
    E: int
    k: int
    I_moe: int
    I_dense: int
    I_shared: int
    nh: int
    nkv: int
    d_qk: int
    d_v: int
    kv_lora: int = 0
    q_lora: int = 0
    d_rope: int = 0
    first_dense: int = 0
    layer_types: List[str] = field(default_factory=list)
    lin_nk: int = 0
    lin_nv: int = 0
    lin_dk: int = 0
    lin_dv: int = 0
    conv_k: int = 0
    expert_bias: bool = False
    attn_bias: bool = False
    attn_gate: bool = False
    tie: bool = False

    @staticmethod
    def from_config(cfg: Dict) -> "ModelDims":
        g = cfg.get
        mt = g("model_type", "qwen3_moe")
        H, L, V = g("hidden_size"), g("num_hidden_layers"), g("vocab_size")
        nh, nkv = g("num_attention_heads"), g("num_key_value_heads") or g("num_attention_heads")
        hd = g("head_dim") or H // nh
        d = ModelDims(model_type=mt, H=H, L=L, V=V, E=0, k=g("num_experts_per_tok", 1), I_moe=0, I_dense=0, I_shared=0,
                      nh=nh, nkv=nkv, d_qk=hd, d_v=hd, tie=bool(g("tie_word_embeddings", False)),
                      attn_bias=bool(g("attention_bias", False)))
        if mt.startswith("deepseek"):
            d.E, d.I_moe, d.I_dense = g("n_routed_experts"), g("moe_intermediate_size"), g("intermediate_size")
            d.I_shared = (g("n_shared_experts") or 0) * d.I_moe
            d.kv_lora, d.q_lora = g("kv_lora_rank"), g("q_lora_rank") or 0
            d.d_rope = g("qk_rope_head_dim")
            d.d_qk, d.d_v = g("qk_nope_head_dim") + d.d_rope, g("v_head_dim")
            d.first_dense = g("first_k_dense_replace", 0)
            d.layer_types = ["mla"] * L
        elif mt.startswith("gpt_oss"):
            d.E, d.I_moe = g("num_local_experts"), g("intermediate_size")
            d.expert_bias = True
            d.layer_types = ["gqa"] * L
        elif mt.startswith("qwen3_5"):
            d.E, d.I_moe = g("num_experts"), g("moe_intermediate_size")
            d.I_shared = g("shared_expert_intermediate_size", 0)
            d.lin_nk, d.lin_nv = g("linear_num_key_heads"), g("linear_num_value_heads")
            d.lin_dk, d.lin_dv = g("linear_key_head_dim"), g("linear_value_head_dim")
            d.conv_k = g("linear_conv_kernel_dim", 4)
            d.attn_gate = bool(g("attn_output_gate", True))
            lt = g("layer_types") or [("full_attention" if (i + 1) % g("full_attention_interval", 4) == 0 else "linear_attention") for i in range(L)]
            d.layer_types = ["gated_gqa" if t == "full_attention" else "linear" for t in lt]
        else:
            d.E, d.I_moe = g("num_experts"), g("moe_intermediate_size")
            d.layer_types = ["gqa"] * L
        return d

    @staticmethod
    def from_json(path: Path) -> "ModelDims":
        cfg = json.load(open(path))
        return ModelDims.from_config(cfg.get("text_config", cfg))

    # -------------------------------------------------------------------------------------- parameter counts
    def attn_params(self, kind: str) -> int:
        H = self.H
        if kind == "mla":
            q = H * self.nh * self.d_qk if not self.q_lora else H * self.q_lora + self.q_lora + self.q_lora * self.nh * self.d_qk
            kv = H * (self.kv_lora + self.d_rope) + self.kv_lora + self.kv_lora * self.nh * (self.d_qk - self.d_rope + self.d_v)
            return q + kv + self.nh * self.d_v * H
        if kind == "linear":
            kd, vd = self.lin_nk * self.lin_dk, self.lin_nv * self.lin_dv
            conv = (2 * kd + vd) * self.conv_k
            return H * (2 * kd + 2 * vd) + 2 * H * self.lin_nv + conv + 2 * self.lin_nv + self.lin_dv + vd * H
        qo = self.nh * self.d_qk
        n = H * qo * (2 if kind == "gated_gqa" else 1) + 2 * H * self.nkv * self.d_qk + qo * H
        if kind in ("gqa", "gated_gqa") and not self.model_type.startswith("gpt_oss"):
            n += 2 * self.d_qk  # q/k norm
        if self.attn_bias:
            n += qo + 2 * self.nkv * self.d_qk + H
        if self.model_type.startswith("gpt_oss"):
            n += self.nh  # sinks
        return n

    def layer_shape(self, idx: int) -> LayerShape:
        H = self.H
        kind = "dense" if idx < self.first_dense else "moe"
        ak = self.layer_types[idx]
        per_expert = 3 * H * self.I_moe + ((2 * self.I_moe + H) if self.expert_bias else 0)
        router = H * self.E + (self.E if self.expert_bias else 0)
        shared = 3 * H * self.I_shared + (H if (self.I_shared and self.model_type.startswith("qwen3_5")) else 0)
        return LayerShape(kind=kind, attn_kind=ak, attn_params=self.attn_params(ak),
                          expert_params_per_expert=per_expert if kind == "moe" else 0,
                          dense_mlp_params=3 * H * self.I_dense if kind == "dense" else 0,
                          shared_params=shared if kind == "moe" else 0, router_params=router if kind == "moe" else 0,
                          norm_params=2 * H)


@dataclass
class StaticMemory:
    """Bytes resident for the whole step, by category."""

    params: int = 0
    grads: int = 0
    optimizer_device: int = 0
    optimizer_host: int = 0
    fp8_weights: int = 0
    detail: Dict[str, int] = field(default_factory=dict)

    @property
    def device_total(self) -> int:
        return self.params + self.grads + self.optimizer_device + self.fp8_weights


def chunk_layers(dims: ModelDims, par: ParallelCfg, pp_rank: int) -> Tuple[range, range]:
    """Layer ids of the rank's two pipeline chunks (stage ``r`` and stage ``2·pp−1−r``)."""
    S = 2 * par.pp
    return layer_partition(dims.L, S, pp_rank), layer_partition(dims.L, S, S - 1 - pp_rank)


def static_memory(dims: ModelDims, par: ParallelCfg, pp_rank: int) -> StaticMemory:
    c0, c1 = chunk_layers(dims, par, pp_rank)
    dense = expert = quantised = 0
    for idx in list(c0) + list(c1):
        ls = dims.layer_shape(idx)
        dense += ls.attn_params + ls.dense_mlp_params + ls.shared_params + ls.router_params + ls.norm_params
        expert += ls.expert_params_per_expert * (dims.E // par.ep)
        # projections and expert matrices take the fp8 path; routers, norms, embedding and lm_head stay bf16
        quantised += ls.attn_params + ls.dense_mlp_params + ls.shared_params + ls.expert_params_per_expert * (dims.E // par.ep)
    edge = 0
    if pp_rank == 0:
        edge += dims.V * dims.H  # embedding on the first stage
        edge += dims.H + (0 if dims.tie else dims.V * dims.H)  # final norm + lm_head on the last stage (same rank in a V)
    dense += edge
    gb, mb = DTYPE_BYTES[par.grad_dtype], DTYPE_BYTES[par.momentum_dtype]
    out = StaticMemory()
    out.params = 2 * (dense + expert)
    if par.reshard_params:
        # while a step runs the flat buffers are whole and the owned parameters exist a second time; between steps only
        # the owned copy stays (the estimate is the peak inside a step)
        out.params += int(2 * (dense / (par.dp * par.cp * par.ep) + expert / (par.dp * par.cp)))
    out.grads = gb * (dense + expert)
    if par.fp8_training:
        # one e4m3 byte per element in each orientation (forward reads W, the input gradient reads W^T), cached for the
        # whole step; the fp32 scales add 1/4096 of that
        out.fp8_weights = int(2 * quantised * (1 + 4 / (128 * 128)))
    dense_owned = dense / (par.dp * par.cp * par.ep)
    expert_owned = expert / (par.dp * par.cp)
    if par.optimizer == "adamw":
        state = 8 * (dense_owned + expert_owned)  # two fp32 moments
    else:
        # Muon momentum for matrices; embedding, lm_head, router, norms and biases use AdamW (two fp32 moments)
        adam_elems = edge / (par.dp * par.cp * par.ep)
        state = mb * (dense_owned - adam_elems + expert_owned) + 8 * adam_elems
    state = int(state)
    if par.offload_optimizer_state:
        resident = min(state, int(par.resident_state_gb * (1 << 30)))
        out.optimizer_host = state - resident
        out.optimizer_device = resident + 3 * 512 * 1024 * 1024  # + staging buffers of the host-offloaded part
    else:
        out.optimizer_device = state
    out.detail = {"dense_param_elems": int(dense), "expert_param_elems": int(expert), "edge_param_elems": int(edge)}
    return out
