"""Distributed runtime setup: process group, fail-fast hooks and the (pp, dp, cp, ep) mesh.

One process per GPU, ``torch.distributed`` with the NCCL backend for bootstrap, pipeline p2p and
scalar reductions; CPU runs (tests, the tiny-model oracle) use gloo. Mirrors the public surface of
pithtrain/modules/distributed.py:17-170 (``DistributedCfg``, ``setup_distributed``).
"""

from __future__ import annotations

import atexit
import os
import sys
import threading
from dataclasses import dataclass
from datetime import timedelta
from typing import Literal, Optional

import torch
import torch.distributed as dist

from ..config import SlottedDefault
from ..contexts import distributed
from ..parallel.mesh import Mesh4D


@dataclass(init=False, slots=True)
class DistributedCfg(SlottedDefault):
    """Parallelism degrees (PP, CP, EP), sharding strategy and collective timeout; DP is inferred."""

    pipeline_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_parallel_size: int = 1
    timeout: timedelta = timedelta(minutes=15)
    sharding_strategy: Literal["fsdp", "hsdp"] = "fsdp"
    reshard_params: bool = False
    """Shard the parameters too between steps: after the gradient reduction a rank keeps only the parameters it owns
    and the next step starts with one all-gather per shard group (the reference's FSDP2 setting, where resharding is
    switched off inside a pipeline step). Off by default: with 180 GB per GPU the parameters stay resident and the
    updated regions are published by peer stores. Uses the NCCL shard collectives."""
    backend: str = "auto"
    """"auto" picks nccl when CUDA is available and gloo otherwise."""
    ep_backend: Literal["auto", "nccl", "fused"] = "auto"
    """Expert-parallel transport: NCCL all-to-all (baseline) or the fused peer-memory kernels."""
    shard_backend: Literal["auto", "nccl"] = "auto"
    """Gradient reduce-scatter and parameter publication of a shard group: kernels over peer memory on one node
    ("auto"), or NCCL always (the baseline, and what groups that span nodes use anyway)."""
    cp_backend: Literal["auto", "nccl"] = "auto"
    """Context-parallel ring: publish-and-pull over peer memory ("auto") or hop-by-hop NCCL send/recv."""
    ep_capacity_factor: Optional[float] = None
    """Receive capacity of the fused expert-parallel transport. None (default): the exact worst case, ``ep * m`` rows
    per micro-batch of ``m`` tokens, which no routing can overflow. A number opts into a smaller buffer of that
    multiple of the expected de-duplicated volume; an overflow then fails the step loudly (status word)."""
    peer_wait_timeout: timedelta = timedelta(seconds=60)
    """Limit of every in-kernel wait on another GPU's flag (peer-memory transports). A wait that runs out sets the
    device status word; the train step reads it once per step and every rank raises ``KernelStatusError`` before
    the step's result is kept. Long enough for a rank stalled in data loading or first-step initialisation."""


def setup_torch_runtime() -> None:
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.set_float32_matmul_precision("high")


def setup_default_process_group(cfg: DistributedCfg) -> None:
    """Initialise the default process group from torchrun-style environment variables.

    Without ``RANK`` in the environment a single-process world is assumed (no process group is
    created), which is what unit tests and 1-GPU runs use.
    """
    use_cuda = torch.cuda.is_available()
    backend = cfg.backend
    if backend == "auto":
        backend = "nccl" if use_cuda else "gloo"
    distributed.backend = backend
    distributed.rank = int(os.environ.get("RANK", "0"))
    distributed.world_size = int(os.environ.get("WORLD_SIZE", "1"))
    distributed.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    distributed.local_world_size = int(os.environ.get("LOCAL_WORLD_SIZE", str(distributed.world_size)))

    if backend == "nccl":
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
        os.environ.setdefault("TORCH_NCCL_BLOCKING_WAIT", "0")
        os.environ.setdefault("TORCH_NCCL_DUMP_ON_TIMEOUT", "1")
        os.environ["TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC"] = str(int(cfg.timeout.total_seconds()))
        torch.cuda.set_device(distributed.local_rank)
        distributed.device = torch.device("cuda", distributed.local_rank)
        from .. import _native

        if _native.available():
            _native.set_peer_wait_limit(cfg.peer_wait_timeout.total_seconds())
    else:
        distributed.device = torch.device("cuda", distributed.local_rank) if use_cuda and backend != "gloo" else torch.device("cpu")

    if "RANK" in os.environ and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = dict(backend=backend, timeout=cfg.timeout)
        if backend == "nccl":
            kwargs["device_id"] = distributed.device
        dist.init_process_group(**kwargs)
        atexit.register(_destroy)


def _destroy() -> None:
    try:
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


def setup_failfast_excepthook() -> None:
    """Hard-exit on an uncaught exception so peers fail fast instead of waiting on this rank.

    The default shutdown drains in-flight collectives that the other ranks may never complete;
    ``os._exit`` skips that drain (same policy as pithtrain/modules/distributed.py:103-126).
    """
    original = sys.excepthook

    def excepthook(exc_type, exc_value, exc_tb, *_):
        try:
            original(exc_type, exc_value, exc_tb)
        except Exception:
            pass
        try:
            sys.stdout.flush()
            sys.stderr.flush()
        except Exception:
            pass
        os._exit(1)

    sys.excepthook = excepthook
    threading.excepthook = lambda args: excepthook(args.exc_type, args.exc_value, args.exc_traceback)


def setup_device_mesh(cfg: DistributedCfg) -> None:
    pp, cp, ep = cfg.pipeline_parallel_size, cfg.context_parallel_size, cfg.expert_parallel_size
    world, divisor = distributed.world_size, pp * cp * ep
    if world % divisor != 0:
        raise RuntimeError(f"world_size={world} not divisible by pp={pp} * cp={cp} * ep={ep}")
    if ep > 32:
        raise RuntimeError("expert_parallel_size must be <= 32 (destination bitmask is 32 bits)")
    dp = world // divisor
    mesh = Mesh4D(pp=pp, dp=dp, cp=cp, ep=ep, rank=distributed.rank)
    mesh.build_groups(timeout=cfg.timeout)
    distributed.device_mesh = mesh
    c = mesh.coords()
    distributed.pp_size, distributed.pp_rank, distributed.pp_group = pp, c["pp"], mesh.group("pp")
    distributed.dp_size, distributed.dp_rank, distributed.dp_group = dp, c["dp"], mesh.group("dp")
    distributed.cp_size, distributed.cp_rank, distributed.cp_group = cp, c["cp"], mesh.group("cp")
    distributed.ep_size, distributed.ep_rank, distributed.ep_group = ep, c["ep"], mesh.group("ep")
    distributed.dp_cp_group = mesh.group("dp", "cp")
    distributed.dp_cp_ep_group = mesh.group("dp", "cp", "ep")
    distributed.dp_ep_group = mesh.group("dp", "ep")


def setup_distributed(cfg: object, failfast: bool = True) -> None:
    """Initialise the distributed runtime: process group, fail-fast hook and device mesh."""
    assert hasattr(cfg, "distributed") and isinstance(cfg.distributed, DistributedCfg)
    setup_torch_runtime()
    setup_default_process_group(cfg.distributed)
    if failfast and "RANK" in os.environ and os.environ.get("PITHTRAIN_NO_FAILFAST") != "1":
        setup_failfast_excepthook()
    distributed.shard_backend, distributed.cp_backend = cfg.distributed.shard_backend, cfg.distributed.cp_backend
    setup_device_mesh(cfg.distributed)
