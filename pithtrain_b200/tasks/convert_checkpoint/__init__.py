"""Checkpoint conversion between Hugging Face safetensors and the framework's canonical DCP layout.

``launch(ConvertCheckpointCfg)`` runs one direction (``hf2dcp`` or ``dcp2hf``); model families whose Hugging Face
key layout differs from the in-memory one register a :class:`ModelConverter` in :data:`CONVERTERS`.
"""

from ._registry import CONVERTERS, ModelConverter
from ._core import ConvertCheckpointCfg, launch, hf2dcp, dcp2hf

__all__ = ["ConvertCheckpointCfg", "launch", "hf2dcp", "dcp2hf", "CONVERTERS", "ModelConverter"]
