"""Qwen3.5-MoE checkpoints: multimodal wrapper names and fused expert tensors.

Import keeps ``model.language_model.*`` (and ``lm_head.*``), drops the vision tower and multi-token
prediction heads, and splits the fused ``mlp.experts.{gate_up_proj,down_proj}`` stacks into one
``....experts.<e>.<proj>.weight`` entry per expert. Export re-nests everything under
``model.language_model``. Behaviour of pithtrain/tasks/convert_checkpoint/qwen35_moe.py:27-140.
"""

from __future__ import annotations

import re
from typing import Dict, Iterable

import torch

from ._registry import ModelConverter, register

_LM = "model.language_model."
_DROP = ("model.visual.", "mtp.", "model.mtp.")
_FUSED_RE = re.compile(r"(.*\.mlp\.experts)\.(gate_up_proj|down_proj)$")
_SPLIT_RE = re.compile(r"(.*\.mlp\.experts)\.(\d+)\.(gate_up_proj|down_proj)\.weight$")


class Qwen35MoeConverter(ModelConverter):
    name = "qwen3_5_moe"
    model_types = ("qwen3_5_moe", "qwen3_5_moe_text")

    def detect_canonical(self, keys: Iterable[str]) -> bool:
        keys = list(keys)
        return any(".linear_attn." in k for k in keys) and any(_SPLIT_RE.match(k) for k in keys)

    def import_tensors(self, hf: Dict[str, torch.Tensor], config: dict) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for key, t in hf.items():
            if key.startswith(_DROP):
                continue
            if key.startswith(_LM):
                name = key[len(_LM):]
            elif key.startswith("lm_head."):
                name = key
            else:
                name = key.removeprefix("model.")
            m = _FUSED_RE.match(name)
            if m is not None and t.dim() == 3:
                for e in range(t.shape[0]):
                    out[f"{m.group(1)}.{e}.{m.group(2)}.weight"] = t[e].contiguous()
            else:
                out[name] = t
        return out

    def export_tensors(self, canonical: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        stacks: Dict[str, Dict[int, torch.Tensor]] = {}
        for k, v in canonical.items():
            m = _SPLIT_RE.match(k)
            if m is not None:
                stacks.setdefault(f"{m.group(1)}.{m.group(3)}", {})[int(m.group(2))] = v
            elif k.startswith("lm_head."):
                out[k] = v
            else:
                out[_LM + k] = v
        for base, by_idx in stacks.items():
            out[_LM + base] = torch.stack([by_idx[i] for i in range(len(by_idx))])
        return out


register(Qwen35MoeConverter())
