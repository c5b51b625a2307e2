"""Checkpoint conversion task: Hugging Face safetensors <-> canonical DCP."""
from ._core import ConvertCheckpointCfg, dcp2hf, hf2dcp, launch  # noqa: F401
from ._registry import CONVERTERS, ModelConverter  # noqa: F401
