"""Throughput benchmark recipes: one table instead of one file per mesh.

Every recipe is the reference's benchmark protocol — Muon, constant learning rate 1e-6, 25 steps,
force-balanced routing (``benchmark=True``), micro-batch 1, global batch 1024 sequences unless noted
(benchmarks/pretraining/qwen3-30b-a3b/setup.py:39-52 and the per-mesh scripts beside it in the reference) —
plus single-node B200 meshes sized for 180 GB per GPU. A recipe name is ``<cluster>/<mesh>``, e.g.
``b200-1n8g/pp2-dp1-cp1-ep4-seq4096-bf16``; the mesh string is parsed, so new meshes need no new code.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List

from pithtrain_b200.modules.training import make_constant_scheduler, make_muon_optimizer
from pithtrain_b200.tasks.pretrain_lm import PretrainLMCfg

ROOT = Path(__file__).resolve().parents[2]
YARN_GPT_OSS = {"rope_scaling": {"rope_type": "yarn", "factor": 32.0, "beta_fast": 32.0, "beta_slow": 1.0,
                                 "original_max_position_embeddings": 4096, "truncate": False},
                "rope_theta": 150000, "initial_context_length": 4096, "max_position_embeddings": 131072}


@dataclass
class ModelRecipe:
    config: str  # example directory that holds config.json
    tokens: str  # sub-directory of workspace/datasets/dclm-baseline/toktxt
    lb_type: str
    lb_coef: float = 1e-3
    overrides: Dict = field(default_factory=dict)
    meshes: List[str] = field(default_factory=list)


MODELS: Dict[str, ModelRecipe] = {
    "qwen3-30b-a3b": ModelRecipe("qwen3-30b-a3b", "qwen3", "global-batch", meshes=[
        "b200-1n1g/pp1-dp1-cp1-ep1-seq4096-bf16-gbs32", "b200-1n2g/pp1-dp1-cp1-ep2-seq4096-bf16-gbs64",
        "b200-1n4g/pp1-dp1-cp1-ep4-seq4096-bf16-gbs128", "b200-1n8g/pp2-dp1-cp1-ep4-seq4096-bf16-gbs256",
        "b200-1n8g/pp2-dp1-cp1-ep4-seq4096-fp8-gbs256",
        "b200-1n8g/pp1-dp1-cp1-ep8-seq4096-bf16", "h100-2n8g/pp2-dp1-cp1-ep8-seq2048-bf16",
        "h100-4n8g/pp4-dp1-cp1-ep8-seq4096-bf16", "h100-8n8g/pp4-dp2-cp1-ep8-seq4096-bf16-hsdp"]),
    "deepseek-v2-lite": ModelRecipe("deepseek-v2-lite", "deepseek-v2", "sequence", 3e-3, meshes=[
        "b200-1n8g/pp1-dp1-cp1-ep8-seq2048-bf16", "b200-1n8g/pp1-dp1-cp1-ep8-seq4096-fp8", "b200-1n8g/pp1-dp1-cp2-ep4-seq8192-bf16",
        "h100-1n8g/pp1-dp1-cp1-ep8-seq2048-bf16"]),
    "gpt-oss-120b": ModelRecipe("gpt-oss-120b", "gpt-oss", "micro-batch", overrides=YARN_GPT_OSS, meshes=[
        "b200-4n8g/pp4-dp1-cp1-ep8-seq2048-bf16", "h100-8n8g/pp8-dp1-cp1-ep8-seq2048-bf16"]),
    "gpt-oss-20b": ModelRecipe("gpt-oss-20b", "gpt-oss", "micro-batch", overrides=YARN_GPT_OSS, meshes=[
        "b200-1n8g/pp1-dp1-cp1-ep8-seq2048-bf16", "b200-1n8g/pp1-dp1-cp4-ep2-seq32768-fp8-gbs64"]),
    "qwen3.5-35b-a3b": ModelRecipe("qwen3.5-35b-a3b", "qwen3.5", "global-batch", meshes=[
        "b200-1n8g/pp1-dp1-cp1-ep8-seq3072-bf16", "h100-2n8g/pp2-dp1-cp1-ep8-seq1536-bf16", "h100-4n8g/pp4-dp1-cp1-ep8-seq3072-bf16"]),
}

_MESH = re.compile(r"pp(\d+)-dp(\d+)-cp(\d+)-ep(\d+)-seq(\d+)-(bf16|fp8)(?:-gbs(\d+))?(-hsdp)?$")


def parse_mesh(name: str) -> Dict:
    m = _MESH.search(name)
    if not m:
        raise ValueError(f"cannot parse mesh name {name!r}")
    pp, dp, cp, ep, seq = (int(x) for x in m.groups()[:5])
    return dict(pp=pp, dp=dp, cp=cp, ep=ep, seq=seq, fp8=m.group(6) == "fp8", gbs=int(m.group(7) or 1024),
                hsdp=bool(m.group(8)), gpus=pp * dp * cp * ep)


def write_model_config(model: str, out_dir: Path) -> Path:
    r = MODELS[model]
    cfg = json.load(open(ROOT / "examples" / "pretrain_lm" / r.config / "config.json"))
    cfg.update(r.overrides)
    out_dir.mkdir(parents=True, exist_ok=True)
    path = out_dir / "model.json"
    path.write_text(json.dumps(cfg, indent=2))
    return path


def make_cfg(model: str, mesh: str, workspace: Path = Path("workspace")) -> PretrainLMCfg:
    r, m = MODELS[model], parse_mesh(mesh)
    cfg = PretrainLMCfg()
    d = cfg.distributed
    d.pipeline_parallel_size, d.expert_parallel_size, d.context_parallel_size = m["pp"], m["ep"], m["cp"]
    if m["hsdp"]:
        d.sharding_strategy = "hsdp"
    t = cfg.training
    t.model = write_model_config(model, workspace / "benchmarks" / model)
    data = workspace / "datasets" / "dclm-baseline" / "toktxt" / r.tokens
    t.dataset = data if data.exists() else None  # falls back to the seeded synthetic token stream
    t.optimizer, t.scheduler, t.lr, t.max_steps = make_muon_optimizer, make_constant_scheduler, 1.0e-6, 25
    t.micro_batch_size, t.global_batch_size, t.sequence_length = 1, m["gbs"], m["seq"]
    t.moe_load_balance_type, t.moe_load_balance_coef = r.lb_type, r.lb_coef
    t.benchmark, t.fp8 = True, m["fp8"]
    t.grad_dtype, t.muon_momentum_dtype = "bf16", "bf16"
    t.offload_optimizer_state = m["gpus"] == 1
    return cfg
