"""GPT-OSS checkpoints: MXFP4 expert weights, stacked experts, ``[E, in, out]`` layout on the hub.

Import: ``*_blocks`` (two FP4 values per byte) and ``*_scales`` (E8M0 exponents, bias 127) are
dequantised to bf16 — value = LUT[nibble] * 2^(scale-127) — giving ``[E, out, in]``; un-quantised
hub checkpoints store ``[E, in, out]`` and are transposed. Stacked tensors are split into one entry
per expert without a ``.weight`` suffix. Export restacks and transposes back. Behaviour of
pithtrain/tasks/convert_checkpoint/gpt_oss.py:15-176.
"""

from __future__ import annotations

import re
from typing import Dict, Iterable

import torch

from ._registry import ModelConverter, canonical_to_hf_name, hf_to_canonical_name, register

FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)
EXPERT_PARAMS = ("gate_up_proj", "gate_up_proj_bias", "down_proj", "down_proj_bias")
_EXPERT_RE = re.compile(r"(.*\.mlp\.experts)\.(\d+)\.(gate_up_proj_bias|down_proj_bias|gate_up_proj|down_proj)$")


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """``blocks[..., G, 16]`` uint8 + ``scales[..., G]`` uint8 -> ``[..., G*32]`` in ``dtype``.

    The low nibble of each byte is the even element, the high nibble the odd one.
    """
    lut = torch.tensor(FP4_VALUES, dtype=torch.float32, device=blocks.device)
    lo, hi = (blocks & 0x0F).long(), (blocks >> 4).long()
    vals = torch.stack([lut[lo], lut[hi]], dim=-1).flatten(-2)  # [..., G, 32]
    exp = scales.to(torch.int32) - 127
    out = torch.ldexp(vals, exp.unsqueeze(-1))
    return out.flatten(-2).to(dtype)


class GptOssConverter(ModelConverter):
    name = "gpt_oss"
    model_types = ("gpt_oss",)

    def detect_canonical(self, keys: Iterable[str]) -> bool:
        return any(_EXPERT_RE.match(k) for k in keys)

    def import_tensors(self, hf: Dict[str, torch.Tensor], config: dict) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        done = set()
        for key, t in hf.items():
            name = hf_to_canonical_name(key)
            if ".mlp.experts." not in name:
                out[name] = t
                continue
            base = name
            for suf in ("_blocks", "_scales"):
                if base.endswith(suf):
                    base = base[: -len(suf)]
            if base in done:
                continue
            done.add(base)
            hkey = canonical_to_hf_name(base)
            if hkey + "_blocks" in hf:  # MXFP4: rows are outputs already
                full = dequant_mxfp4(hf[hkey + "_blocks"], hf[hkey + "_scales"])
            else:
                full = hf[hkey]
                if full.dim() == 3:  # hub layout [E, in, out] -> [E, out, in]
                    full = full.transpose(1, 2).contiguous()
            prefix, pname = base.rsplit(".", 1)
            for e in range(full.shape[0]):
                out[f"{prefix}.{e}.{pname}"] = full[e].contiguous()
        return out

    def export_tensors(self, canonical: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        stacks: Dict[str, Dict[int, torch.Tensor]] = {}
        for k, v in canonical.items():
            m = _EXPERT_RE.match(k)
            if m is None:
                out[canonical_to_hf_name(k)] = v
            else:
                stacks.setdefault(f"{m.group(1)}.{m.group(3)}", {})[int(m.group(2))] = v
        for base, by_idx in stacks.items():
            full = torch.stack([by_idx[i] for i in range(len(by_idx))])
            if full.dim() == 3:
                full = full.transpose(1, 2).contiguous()
            out[canonical_to_hf_name(base)] = full
        return out


register(GptOssConverter())
