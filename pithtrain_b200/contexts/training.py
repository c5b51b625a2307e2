"""Training runtime state (filled by ``modules.training.setup_training``)."""
from typing import Any

fp8: bool = False
Linear: Any = None
GroupedLinear: Any = None

model: Any = None  # dualpipe.DualPipeV
dataset: Any = None
optimizers: tuple = ()
schedulers: tuple = ()
shard_groups: tuple = ()
model_config: Any = None  # parallel.flat_shard.FlatShardGroup instances

step: int = 0
