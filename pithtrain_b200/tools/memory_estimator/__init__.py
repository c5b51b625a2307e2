"""Analytic peak-memory estimator: ``python -m pithtrain_b200.tools.memory_estimator --help``."""
from .model_profile import ModelDims, ParallelCfg, static_memory  # noqa: F401
from .schedule_simulator import Estimate, estimate  # noqa: F401
