"""Training setup: configuration, model construction, flat parameter sharding, optimizers and
learning-rate schedules.

``setup_training(cfg)`` seeds the RNGs, opens the dataset, builds the two pipeline chunks of this
rank, initialises weights, places every parameter into the flat shard groups
(:mod:`pithtrain_b200.parallel.flat_shard`), attaches load-balance losses, wraps the chunks in
``DualPipeV`` and calls the user-supplied optimizer and scheduler builders — the flow of
pithtrain/modules/training.py:379-478 with the framework's own sharding in place of FSDP2.
"""

from __future__ import annotations

import json
import math
import random
from dataclasses import dataclass
from pathlib import Path
from types import SimpleNamespace
from typing import Any, Callable, Literal, Optional, Union

import numpy as np
import torch
import torch.nn as nn
from torch.optim import Optimizer
from torch.optim.lr_scheduler import LambdaLR, LRScheduler

from ..config import SlottedDefault
from ..contexts import distributed, training
from ..dualpipe.comm import set_p2p_tensor_dtype, set_p2p_tensor_shapes
from ..modules.dataset import ConcatDataset, MemmapDataset, SyntheticDataset
from ..modules.load_balance import force_balance, make_load_balance_loss_fn
from ..modules.optimizer import AdamW, Muon
from ..parallel import ep as ep_mod
from ..parallel.flat_shard import build_shard_groups


def is_muon_param(name: str, param: torch.Tensor) -> bool:
    """True when Muon should optimise ``param``: 2-D hidden weights and stacked 3-D expert weights.

    1-D parameters, biases (also stacked ``*_bias``), embeddings, the LM head and MoE routers go to
    AdamW (same split as pithtrain/modules/training.py:40-57).
    """
    if param.ndim < 2:
        return False
    if name.endswith(".bias") or name.endswith("_bias"):
        return False
    if name.endswith("embed_tokens.weight") or name.endswith("lm_head.weight"):
        return False
    if ".gate.weight" in name or ".router.weight" in name:
        return False
    return True


def make_muon_optimizer(cfg: "TrainingCfg", *, weight_decay: float = 0.1) -> tuple[Optimizer, ...]:
    muon_params, adamw_params = [], []
    for name, p in training.model.named_parameters():
        if not p.requires_grad:
            continue
        (muon_params if is_muon_param(name, p) else adamw_params).append(p)
    mdt = {"fp32": torch.float32, "bf16": torch.bfloat16}[cfg.muon_momentum_dtype]
    return (Muon(muon_params, lr=cfg.lr, weight_decay=weight_decay, momentum_dtype=mdt,
                 offload_state=cfg.offload_optimizer_state,
                 device_state_budget=int(cfg.optimizer_device_state_gb * (1 << 30))),
            AdamW(adamw_params, lr=cfg.lr, weight_decay=weight_decay))


def make_adamw_optimizer(cfg: "TrainingCfg", *, weight_decay: float = 0.1) -> tuple[Optimizer, ...]:
    return (AdamW([p for p in training.model.parameters() if p.requires_grad], lr=cfg.lr, weight_decay=weight_decay),)


def wsd_lambda(max_steps: int, lr: float, start_lr: float = 0.0, warmup_ratio: float = 0.0, final_lr: float = 0.0,
               decay_ratio: float = 0.1, decay_shape: str = "cosine") -> Callable[[int], float]:
    if decay_shape not in ("cosine", "linear"):
        raise ValueError(f"Unknown decay_shape: {decay_shape!r}")
    if warmup_ratio + decay_ratio > 1:
        raise ValueError("warmup_ratio + decay_ratio must be <= 1")
    warmup, decay = round(warmup_ratio * max_steps), round(decay_ratio * max_steps)
    stable = max_steps - warmup - decay
    f0, f1 = start_lr / lr, final_lr / lr

    def fn(step: int) -> float:
        if step < warmup:
            return f0 + (1 - f0) * (step / warmup)
        if decay == 0 or step < warmup + stable:
            return 1.0
        t = min((step - warmup - stable) / decay, 1.0)
        if decay_shape == "cosine":
            return f1 + (1 - f1) * 0.5 * (1 + math.cos(math.pi * t))
        return 1.0 + (f1 - 1.0) * t

    return fn


def make_wsd_scheduler(cfg: "TrainingCfg", *, start_lr: float = 0.0, warmup_ratio: float = 0.0, final_lr: float = 0.0,
                       decay_ratio: float = 0.1, decay_shape: Literal["cosine", "linear"] = "cosine"
                       ) -> tuple[LRScheduler, ...]:
    """Warmup-stable-decay: linear warmup, hold, then cosine or linear decay to ``final_lr``."""
    fn = wsd_lambda(cfg.max_steps, cfg.lr, start_lr, warmup_ratio, final_lr, decay_ratio, decay_shape)
    return tuple(LambdaLR(opt, fn) for opt in training.optimizers)


def make_constant_scheduler(cfg: "TrainingCfg") -> tuple[LRScheduler, ...]:
    return tuple(LambdaLR(opt, lambda _: 1.0) for opt in training.optimizers)


@dataclass(init=False, slots=True)
class TrainingCfg(SlottedDefault):
    dataset: Optional[Path] = None
    """Directory of tokenized ``*.bin`` shards; ``None`` selects the synthetic uniform-token stream."""
    sequence_length: int
    seed: int = 1234
    lr: float
    max_steps: int
    micro_batch_size: int
    global_batch_size: int
    optimizer: Callable[["TrainingCfg"], tuple[Optimizer, ...]]
    scheduler: Callable[["TrainingCfg"], tuple[LRScheduler, ...]]
    model: Union[Path, str, dict]
    """Path to an HF-style ``config.json`` (or its directory), a known model id, or a config dict."""
    save_interval: Optional[int] = None
    save_location: Optional[Path] = None
    moe_load_balance_coef: float = 0.0
    moe_load_balance_type: Literal["micro-batch", "global-batch", "sequence"] = "micro-batch"
    benchmark: bool = False
    fp8: bool = False
    init_std: float = 0.02
    depth_scaled_init: bool = True
    """Scale ``o_proj``/``down_proj`` init by ``1/sqrt(2*num_layers)`` (the reference's default)."""
    nsys_start: Optional[int] = None
    nsys_stop: Optional[int] = None
    memory_profile_start: Optional[int] = None
    memory_profile_stop: Optional[int] = None
    memory_profile_output: Path = Path.cwd()
    # --- additions of this framework -------------------------------------------------------------
    param_dtype: Literal["bf16", "fp32"] = "bf16"
    grad_dtype: Literal["fp32", "bf16"] = "fp32"
    """dtype of the flat gradient accumulators (fp32 matches the reference's reduce dtype)."""
    muon_momentum_dtype: Literal["fp32", "bf16"] = "fp32"
    offload_optimizer_state: bool = False
    """Keep Muon momentum in pinned host memory and stream it through the GPU during the step."""
    optimizer_device_state_gb: float = 0.0
    """With ``offload_optimizer_state``: GiB of Muon momentum that stay on the device anyway."""
    max_grad_norm: float = 1.0
    expert_grad_scaling: Literal["global-mean", "reference"] = "global-mean"
    """``global-mean``: every parameter sees the gradient of the same global token-mean loss, whatever the mesh.
    ``reference``: expert gradients are averaged over dp x cp only, so they are ``ep`` times larger than in a run
    without expert parallelism — what FSDP2's per-mesh averaging gives the reference
    (pithtrain/modules/training.py:341-342); use it to reproduce the reference's loss curves at ``ep > 1``."""
    pair_expert_wgrads: bool = False
    """Compute the expert weight gradients of two consecutive micro-batches in one launch per weight: halves the
    passes over the expert gradient buffers; holds one extra micro-batch of expert activations per layer."""
    num_hidden_layers_override: Optional[int] = None
    """Truncate the model (tests and smoke runs only)."""
    pipeline_overlap: bool = True


KNOWN_MODELS = {
    "Qwen/Qwen3-30B-A3B": "qwen3-30b-a3b",
    "deepseek-ai/DeepSeek-V2-Lite": "deepseek-v2-lite",
    "openai/gpt-oss-20b": "gpt-oss-20b",
    "openai/gpt-oss-120b": "gpt-oss-120b",
    "Qwen/Qwen3.5-35B-A3B": "qwen3.5-35b-a3b",
}


def load_model_config(model: Union[Path, str, dict]) -> SimpleNamespace:
    """Read a model architecture description into a namespace (no network, no transformers needed)."""
    if isinstance(model, dict):
        d = dict(model)
    else:
        key = str(model)
        if key in KNOWN_MODELS:
            path = Path(__file__).resolve().parents[2] / "examples" / "pretrain_lm" / KNOWN_MODELS[key] / "config.json"
        else:
            path = Path(model)
            if path.is_dir():
                path = path / "config.json"
        with open(path) as f:
            d = json.load(f)
    if "text_config" in d and isinstance(d["text_config"], dict):
        inner = dict(d["text_config"])
        inner.setdefault("model_type", d.get("model_type", "") + "_text")
        d = inner
    return SimpleNamespace(**d)


def model_class_for(config: Any):
    from ..models import MODEL_CLASSES

    mt = getattr(config, "model_type", None)
    if mt not in MODEL_CLASSES:
        raise ValueError(f"Unsupported model_type: {mt}")
    return MODEL_CLASSES[mt]


def setup_dataset(cfg: TrainingCfg) -> None:
    if cfg.dataset is None:
        mc = load_model_config(cfg.model)
        training.dataset = SyntheticDataset(mc.vocab_size, cfg.sequence_length, cfg.seed)
        return
    shards = [MemmapDataset(f, cfg.sequence_length) for f in sorted(Path(cfg.dataset).rglob("*.bin"))]
    training.dataset = ConcatDataset(shards, cfg.seed)


def init_weights(model: nn.Module, num_layers: int, init_std: float = 0.02, depth_scaled: bool = True,
                 seed: int = 0, expert_offset: int = 0) -> None:
    """N(0, init_std) for matrices; ``o_proj``/``down_proj`` get ``init_std/sqrt(2*num_layers)`` when
    ``depth_scaled``; 1-D parameters are left as constructed.

    The draw is a function of (seed, parameter name, global expert index) only, so the initial model
    is the same whatever the pipeline / expert / data-parallel layout, replicas agree without a
    broadcast, and experts on different ranks do not start as copies of one another. ``expert_offset``
    is the global index of this rank's first local expert. (The reference draws from the rank's RNG
    stream in module order, pithtrain/modules/training.py:297-325.)
    """
    import zlib

    out_std = init_std / math.sqrt(2.0 * num_layers) if depth_scaled else init_std
    gens = {}

    def gen_for(device) -> torch.Generator:
        key = str(device)
        if key not in gens:
            gens[key] = torch.Generator(device=device)
        return gens[key]

    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() < 2:
                continue
            std = out_std if ("o_proj" in name or "down_proj" in name) else init_std
            g = gen_for(p.device)
            base = (int(seed) * 1000003 + zlib.crc32(name.encode())) % (1 << 62)
            if ".experts." in name and p.dim() >= 2 and "shared" not in name:
                for e in range(p.shape[0]):
                    g.manual_seed(base * 4099 + expert_offset + e + 1)
                    p[e].normal_(mean=0.0, std=std, generator=g)
            else:
                g.manual_seed(base * 4099)
                p.normal_(mean=0.0, std=std, generator=g)


def _num_experts(config) -> int:
    for key in ("num_experts", "n_routed_experts", "num_local_experts"):
        v = getattr(config, key, None)
        if v:
            return int(v)
    return 0


def materialize_small_params(model: nn.Module) -> None:
    """Fill 1-D parameters of a model that was built on the meta device and then bound to real
    storage: ``_init_fill`` (norm scales) or a custom ``_init_fn``, zeros otherwise."""
    with torch.no_grad():
        for _, p in model.named_parameters():
            fn = getattr(p, "_init_fn", None)
            if fn is not None:
                fn(p)
            elif p.dim() < 2:
                p.fill_(getattr(p, "_init_fill", 0.0))


def apply_fsdp(modules: nn.Sequential, sharding_strategy: str = "fsdp", grad_dtype: torch.dtype = torch.float32,
               expert_grad_divisor: Optional[int] = None, reshard_params: bool = False):
    """Place the parameters of both chunks into flat shard groups (experts over dp×cp, the rest over
    dp×cp×ep). ``hsdp`` shards inside cp(×ep) and replicates over dp. ``expert_grad_divisor`` (default ``ep``)
    divides the expert gradients on top of the shard-group average; 1 reproduces the reference's scaling."""
    d = distributed
    if expert_grad_divisor is None:
        expert_grad_divisor = d.ep_size
    mesh = d.device_mesh
    groups = []
    for i, m in enumerate(modules):
        if sharding_strategy == "fsdp" or mesh is None or d.dp_size == 1:
            kw = dict(expert_group=d.dp_cp_group, expert_group_size=d.dp_size * d.cp_size,
                      expert_group_rank=(mesh.local_rank("dp", "cp") if mesh else 0),
                      dense_group=d.dp_cp_ep_group, dense_group_size=d.dp_size * d.cp_size * d.ep_size,
                      dense_group_rank=(mesh.local_rank("dp", "cp", "ep") if mesh else 0))
        elif sharding_strategy == "hsdp":
            cp_ep_group = mesh.ensure_group("cp", "ep")
            kw = dict(expert_group=d.cp_group, expert_group_size=d.cp_size, expert_group_rank=d.cp_rank,
                      dense_group=cp_ep_group, dense_group_size=d.cp_size * d.ep_size,
                      dense_group_rank=mesh.local_rank("cp", "ep"),
                      expert_replica=(d.dp_group, d.dp_size), dense_replica=(d.dp_group, d.dp_size))
        else:
            raise ValueError(f"Unknown sharding_strategy: {sharding_strategy!r}")
        groups.extend(build_shard_groups(m, grad_dtype=grad_dtype, prefix=f"module.{i}.", device=d.device,
                                         expert_grad_divisor=expert_grad_divisor, reshard_params=reshard_params, **kw))
    training.shard_groups = tuple(groups)
    return modules


def setup_model(cfg: TrainingCfg, distributed_cfg: Any) -> None:
    training.fp8 = cfg.fp8
    from ..ops.grouped_linear import GroupedLinear
    from ..ops.linear import Linear

    training.Linear, training.GroupedLinear = Linear, GroupedLinear
    from ..ops import fp8_linear

    fp8_linear.enable(bool(cfg.fp8))
    if cfg.fp8:
        training.Linear, training.GroupedLinear = fp8_linear.FP8Linear, fp8_linear.FP8GroupedLinear

    cp = distributed.cp_size
    config = load_model_config(cfg.model)
    config.max_position_embeddings = cfg.sequence_length
    if cfg.num_hidden_layers_override is not None:
        config.num_hidden_layers = cfg.num_hidden_layers_override
    if cfg.sequence_length % (2 * cp) != 0:
        raise ValueError(f"sequence_length ({cfg.sequence_length}) must be divisible by 2 * context_parallel_size "
                         f"({2 * cp}): zigzag ring attention splits the sequence into 2*cp equal blocks")
    ModelClass = model_class_for(config)
    ep_mod.setup_exchange(getattr(distributed_cfg, "ep_backend", "auto"), getattr(distributed_cfg, "ep_capacity_factor", None))

    dtype = torch.bfloat16 if cfg.param_dtype == "bf16" else torch.float32
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        # parameters are created on the meta device and get their storage from the flat shard
        # groups, so the model is never resident twice
        with torch.device("meta"):
            modules = [ModelClass(config, phase=0), ModelClass(config, phase=1)]
    finally:
        torch.set_default_dtype(prev)
    modules = nn.Sequential(*modules)
    gdt = torch.float32 if cfg.grad_dtype == "fp32" else torch.bfloat16
    apply_fsdp(modules, getattr(distributed_cfg, "sharding_strategy", "fsdp"), gdt,
               expert_grad_divisor=1 if cfg.expert_grad_scaling == "reference" else None,
               reshard_params=bool(getattr(distributed_cfg, "reshard_params", False)))
    for m in modules:
        materialize_small_params(m)
        init_weights(m, config.num_hidden_layers, cfg.init_std, cfg.depth_scaled_init, seed=cfg.seed,
                     expert_offset=distributed.ep_rank * (_num_experts(config) // max(distributed.ep_size, 1)))
    if hasattr(modules[0], "rotary_emb") and hasattr(modules[1], "rotary_emb"):
        modules[1].rotary_emb = modules[0].rotary_emb

    local_seq = cfg.sequence_length // cp
    if cfg.moe_load_balance_coef > 0:
        for m in modules:
            for layer in m.layers.values():
                gate = getattr(layer.mlp, "gate", None) or getattr(layer.mlp, "router", None)
                if gate is None:
                    continue
                fn = make_load_balance_loss_fn(cfg.moe_load_balance_type, cfg.moe_load_balance_coef,
                                               distributed.dp_ep_group, sequence_length=local_seq,
                                               cp_group=distributed.cp_group)
                if hasattr(fn, "init_buffers"):
                    fn.init_buffers(gate.num_experts, gate.weight.device)
                gate.load_balance_loss_fn = fn
    if cfg.benchmark:
        for mod in modules.modules():
            if hasattr(mod, "router_replay"):
                mod.router_replay = force_balance(mod.num_experts)

    from ..dualpipe.dualpipev import DualPipeV

    training.model = DualPipeV(modules)
    training.model.overlap = cfg.pipeline_overlap
    training.model_config = config
    set_p2p_tensor_shapes([(cfg.micro_batch_size, local_seq, config.hidden_size)])
    set_p2p_tensor_dtype(dtype)


def setup_training(cfg: object) -> None:
    """Populate the training context: dataset, model, optimizers, schedulers."""
    assert hasattr(cfg, "training") and isinstance(cfg.training, TrainingCfg)
    t = cfg.training
    training.step = 0
    setup_dataset(t)
    random.seed(t.seed)
    np.random.seed(t.seed)
    torch.manual_seed(t.seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(t.seed)
    setup_model(t, cfg.distributed)
    from ..ops import moe as _moe

    _moe.PAIR_EXPERT_WGRADS = bool(t.pair_expert_wgrads)
    training.optimizers = t.optimizer(t)
    training.schedulers = t.scheduler(t)
    from ..tools.memory_trace import attach_from_env

    attach_from_env(training.model)  # PITHTRAIN_MEMORY_TRACE=<ranks>: one line of memory figures per pipeline action
