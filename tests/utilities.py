"""Helpers shared by the multi-process tests: spawn ``world`` ranks on CPU (gloo) or GPUs (nccl)."""

from __future__ import annotations

import os
import socket
import traceback
from typing import Callable

import torch
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank: int, world: int, port: int, backend: str, fn: Callable, args: tuple, errq) -> None:
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "LOCAL_WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                       "PITHTRAIN_NO_FAILFAST": "1", "TORCHELASTIC_RUN_ID": "pytest"})
    if backend == "gloo":
        os.environ["CUDA_VISIBLE_DEVICES"] = ""
        torch.set_num_threads(1)
    try:
        fn(rank, world, *args)
    except Exception:  # surface the traceback in the parent
        errq.put((rank, traceback.format_exc()))
        raise
    finally:
        import torch.distributed as dist

        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


_FORKSERVER = None


def _context(backend: str):
    """CPU ranks are forked from a server process that has already imported torch (nothing else: no process group, no
    threads), which saves the interpreter start-up and the torch import of every rank of every test; GPU ranks are
    spawned, as CUDA wants."""
    global _FORKSERVER
    if backend != "gloo" or os.environ.get("PITHTRAIN_TEST_SPAWN", "0") == "1":
        return mp.get_context("spawn")
    if _FORKSERVER is None:
        ctx = mp.get_context("forkserver")
        ctx.set_forkserver_preload(["torch", "torch.distributed", "numpy"])
        _FORKSERVER = ctx
    return _FORKSERVER


def launch(world: int, fn: Callable, *args, backend: str = "gloo", timeout: float = 240.0) -> None:
    """Run ``fn(rank, world, *args)`` in ``world`` processes; raises with the first failing rank's traceback."""
    ctx = _context(backend)
    errq = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    failed = None
    for p in procs:
        p.join(timeout)
        if p.is_alive():
            failed = failed or "timeout"
    for p in procs:
        if p.is_alive():
            p.kill()
    if not errq.empty():
        rank, tb = errq.get()
        raise AssertionError(f"rank {rank} failed:\n{tb}")
    bad = [p.exitcode for p in procs if p.exitcode != 0]
    if failed or bad:
        raise AssertionError(f"multi-process test failed: {failed or ''} exit codes {bad}")


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """``1 - 2<x,y>/(|x|^2+|y|^2)``: 0 for identical tensors, insensitive to tiny elements."""
    x, y = x.detach().double(), y.detach().double()
    d = (x * x + y * y).sum()
    return 0.0 if d == 0 else float(1 - 2 * (x * y).sum() / d)
