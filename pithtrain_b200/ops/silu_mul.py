"""``silu(gate) * up`` under the module name of the reference (pithtrain/operators/silu_mul.py:129)."""
from .activations import silu_mul

__all__ = ["silu_mul"]
