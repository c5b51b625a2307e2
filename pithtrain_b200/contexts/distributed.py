"""Distributed runtime state (filled by ``modules.distributed.setup_distributed``)."""
from typing import Any

import torch

rank: int = 0
world_size: int = 1
local_rank: int = 0
local_world_size: int = 1
device: torch.device = torch.device("cpu")
backend: str = "gloo"
# transports of the shard-group collectives and of the context-parallel ring: "auto" = kernels over peer memory when
# the group sits on one node with peer access, NCCL otherwise; "nccl" = always NCCL
shard_backend: str = "auto"
cp_backend: str = "auto"

device_mesh: Any = None  # parallel.mesh.Mesh4D
pp_group: Any = None
dp_group: Any = None
cp_group: Any = None
ep_group: Any = None
# flattened groups used for gradient sharding and statistics
dp_cp_group: Any = None  # shard group of expert parameters
dp_cp_ep_group: Any = None  # shard group of non-expert parameters
dp_ep_group: Any = None  # load-balance statistics

pp_rank: int = 0
pp_size: int = 1
dp_rank: int = 0
dp_size: int = 1
cp_rank: int = 0
cp_size: int = 1
ep_rank: int = 0
ep_size: int = 1


def reset_single_process() -> None:
    """Point every field at a 1-rank world (unit tests that never call setup_distributed)."""
    g = globals()
    g.update(rank=0, world_size=1, local_rank=0, local_world_size=1, backend="gloo", shard_backend="auto", cp_backend="auto",
             device=torch.device("cpu"), device_mesh=None,
             pp_group=None, dp_group=None, cp_group=None, ep_group=None,
             dp_cp_group=None, dp_cp_ep_group=None, dp_ep_group=None,
             pp_rank=0, pp_size=1, dp_rank=0, dp_size=1, cp_rank=0, cp_size=1, ep_rank=0, ep_size=1)
