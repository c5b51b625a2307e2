"""Model-specific checkpoint converters.

A converter recognises a Hugging Face checkpoint (by ``config.json``) or a canonical checkpoint (by
its key set) and rewrites tensors between the two naming/layout schemes. The generic converter
(plain prefix handling) serves models whose Hugging Face checkpoints already store one tensor per
expert (Qwen3-MoE, DeepSeek-V2). Counterpart: pithtrain/tasks/convert_checkpoint/_registry.py:19-40.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterable, List

import torch


def read_hf_config(path: Path) -> dict:
    f = Path(path, "config.json")
    return json.load(open(f)) if f.exists() else {}


def hf_to_canonical_name(key: str) -> str:
    return key if key.startswith("lm_head.") else key.removeprefix("model.")


def canonical_to_hf_name(key: str) -> str:
    return key if key.startswith("lm_head.") else "model." + key


class ModelConverter:
    """Base: identity on tensors, ``model.`` prefix handling on names."""

    name = "generic"
    model_types: tuple = ()

    def detect_hf(self, path: Path) -> bool:
        return read_hf_config(path).get("model_type") in self.model_types

    def detect_canonical(self, keys: Iterable[str]) -> bool:
        return False

    def import_tensors(self, hf: Dict[str, torch.Tensor], config: dict) -> Dict[str, torch.Tensor]:
        """HF names/layout -> canonical names/layout (may consume several inputs per output)."""
        return {hf_to_canonical_name(k): v for k, v in hf.items()}

    def export_tensors(self, canonical: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {canonical_to_hf_name(k): v for k, v in canonical.items()}


CONVERTERS: List[ModelConverter] = []


def register(conv: ModelConverter) -> ModelConverter:
    CONVERTERS.append(conv)
    return conv


def find_for_hf(path: Path) -> ModelConverter:
    for c in CONVERTERS:
        if c.detect_hf(path):
            return c
    return ModelConverter()


def find_for_canonical(keys: Iterable[str]) -> ModelConverter:
    keys = list(keys)
    for c in CONVERTERS:
        if c.detect_canonical(keys):
            return c
    return ModelConverter()
