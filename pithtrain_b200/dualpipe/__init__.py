"""DualPipeV pipeline engine: scheduler, overlapped forward/backward, 5-stage executor."""
from .comm import set_p2p_tensor_dtype, set_p2p_tensor_shapes  # noqa: F401
from .utils import FP8WeightCacheControl, WeightGradStore  # noqa: F401


def __getattr__(name):
    if name == "DualPipeV":
        from .dualpipev import DualPipeV

        return DualPipeV
    raise AttributeError(name)
