"""Training runtime state (filled by ``modules.training.setup_training``)."""
from typing import Any

fp8: bool = False
Linear: Any = None
GroupedLinear: Any = None

model: Any = None  # dualpipe.DualPipeV
dataset: Any = None
optimizers: tuple = ()
schedulers: tuple = ()
shard_groups: tuple = ()  # parallel.flat_shard.FlatShardGroup instances
model_config: Any = None  # the parsed config.json (SimpleNamespace)

step: int = 0
