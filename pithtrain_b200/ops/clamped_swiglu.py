"""GPT-OSS clamped SwiGLU under the module name of the reference (pithtrain/operators/clamped_swiglu.py:148)."""
from .activations import clamped_swiglu

__all__ = ["clamped_swiglu"]
