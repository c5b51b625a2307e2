"""Hugging Face <-> canonical DCP checkpoint conversion and the task entry point.

``hf2dcp`` reads every ``*.safetensors`` shard of a Hugging Face checkpoint, lets the matching
converter map names and layouts to the canonical scheme and writes a model-only DCP directory that
training loads non-strictly. ``dcp2hf`` goes the other way and writes safetensors shards of at most
``max_shard_size`` bytes plus ``model.safetensors.index.json``. Public surface of
pithtrain/tasks/convert_checkpoint/_core.py:29-135.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Literal

import torch

from ...config import SlottedDefault
from ...contexts import logging
from ...modules.logging import LoggingCfg, setup_logging
from . import gpt_oss, qwen35_moe  # noqa: F401  (register converters)
from ._registry import find_for_canonical, find_for_hf, read_hf_config

MODEL_PREFIX = "app.model."


@dataclass(init=False, slots=True)
class ConvertCheckpointCfg(SlottedDefault):
    operation: Literal["hf2dcp", "dcp2hf"]
    load_path: Path
    save_path: Path
    max_shard_size: int = 8 * 1024 ** 3
    logging: LoggingCfg = field(default_factory=LoggingCfg)


def read_safetensors_dir(path: Path, log=None) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    index = Path(path, "model.safetensors.index.json")
    if index.exists():
        files = sorted(set(json.load(open(index))["weight_map"].values()))
    else:
        files = sorted(p.name for p in Path(path).glob("*.safetensors"))
    out: Dict[str, torch.Tensor] = {}
    for i, name in enumerate(files, 1):
        if log:
            log.info("Reading shard %d/%d: %s" % (i, len(files), name))
        with safe_open(str(Path(path, name)), framework="pt", device="cpu") as f:
            for key in f.keys():
                out[key] = f.get_tensor(key)
    return out


def hf2dcp(cfg: ConvertCheckpointCfg, stdout=None) -> int:
    import torch.distributed.checkpoint as dcp

    load_path, save_path = Path(cfg.load_path), Path(cfg.save_path)
    conv = find_for_hf(load_path)
    if stdout:
        stdout.info("hf2dcp with the %s converter: %s" % (conv.name, load_path))
    tensors = conv.import_tensors(read_safetensors_dir(load_path, stdout), read_hf_config(load_path))
    save_path.mkdir(parents=True, exist_ok=True)
    dcp.save({"app": {"model": tensors}}, checkpoint_id=str(save_path), no_dist=True)
    if stdout:
        stdout.info("Saved DCP checkpoint to %s (%d weights)" % (save_path, len(tensors)))
    return len(tensors)


def read_canonical_model(load_path: Path) -> Dict[str, torch.Tensor]:
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader

    md = FileSystemReader(str(load_path)).read_metadata().state_dict_metadata
    flat = {k: torch.empty(tuple(m.size), dtype=m.properties.dtype) for k, m in md.items()
            if k.startswith(MODEL_PREFIX) and hasattr(m, "size")}
    dcp.load(flat, checkpoint_id=str(load_path), no_dist=True)
    return {k[len(MODEL_PREFIX):]: v for k, v in flat.items()}


def plan_shards(tensors: Dict[str, torch.Tensor], max_shard_size: int) -> List[Dict[str, torch.Tensor]]:
    shards: List[Dict[str, torch.Tensor]] = [{}]
    used = 0
    for k, t in tensors.items():
        nbytes = t.numel() * t.element_size()
        if shards[-1] and used + nbytes > max_shard_size:
            shards.append({})
            used = 0
        shards[-1][k] = t
        used += nbytes
    return shards


def dcp2hf(cfg: ConvertCheckpointCfg, stdout=None) -> int:
    from safetensors.torch import save_file

    load_path, save_path = Path(cfg.load_path), Path(cfg.save_path)
    canonical = read_canonical_model(load_path)
    conv = find_for_canonical(canonical.keys())
    if stdout:
        stdout.info("dcp2hf with the %s converter: %d weights from %s" % (conv.name, len(canonical), load_path))
    hf = conv.export_tensors(canonical)
    shards = plan_shards(hf, cfg.max_shard_size)
    save_path.mkdir(parents=True, exist_ok=True)
    weight_map, total = {}, 0
    for i, shard in enumerate(shards):
        name = "model-%05d-of-%05d.safetensors" % (i, len(shards))
        save_file({k: v.contiguous() for k, v in shard.items()}, str(Path(save_path, name)))
        for k, v in shard.items():
            weight_map[k] = name
            total += v.numel() * v.element_size()
    with open(Path(save_path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    if stdout:
        stdout.info("Saved HF checkpoint to %s (%d weights, %d shards)" % (save_path, len(weight_map), len(shards)))
    return len(weight_map)


def launch(cfg: ConvertCheckpointCfg) -> None:
    setup_logging(cfg)
    out = logging.stdout
    out.info("launch(cfg=%s)" % cfg.to_json_dict())
    if cfg.operation == "hf2dcp":
        hf2dcp(cfg, out)
    elif cfg.operation == "dcp2hf":
        dcp2hf(cfg, out)
    else:
        raise ValueError(f"Unknown operation: {cfg.operation!r}")
