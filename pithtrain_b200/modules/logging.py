"""Logging: a rank-filtered stdout logger and optional Weights & Biases tracking.

``logging.stdout.info(msg, rank=0)`` prints on one rank only (``rank=None`` prints everywhere).
wandb is created lazily after the first successful step so failed launches leave no empty runs —
behaviour of pithtrain/modules/logging.py:15-117.
"""

from __future__ import annotations

import logging as pylogging
import os
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

from ..config import SlottedDefault
from ..contexts import distributed, logging

METRICS = (
    "train/step", "train/cross-entropy-loss", "train/load-balance-loss", "train/learning-rate",
    "train/gradient-norm", "infra/tokens-per-second", "infra/peak-gpu-memory", "infra/step-time", "infra/mfu",
)


class StdoutLogger:
    def __init__(self, name: str = "pithtrain_b200") -> None:
        self._logger = pylogging.getLogger(name)
        self._logger.setLevel(pylogging.INFO)
        self._logger.propagate = False
        if not self._logger.handlers:
            h = pylogging.StreamHandler(sys.stdout)
            h.setFormatter(pylogging.Formatter("[%(asctime)s] %(message)s", "%Y-%m-%d %H:%M:%S"))
            self._logger.addHandler(h)

    def _emit(self, level: int, msg: str, rank: Optional[int]) -> None:
        if rank is None or distributed.rank == rank:
            self._logger.log(level, msg)

    def info(self, msg: str, rank: Optional[int] = 0) -> None:
        self._emit(pylogging.INFO, msg, rank)

    def warning(self, msg: str, rank: Optional[int] = 0) -> None:
        self._emit(pylogging.WARNING, msg, rank)

    def error(self, msg: str, rank: Optional[int] = None) -> None:
        self._emit(pylogging.ERROR, msg, rank)


@dataclass(init=False, slots=True)
class LoggingWandbCfg(SlottedDefault):
    entity: str
    project: str
    name: str
    group: Optional[str] = None


@dataclass(init=False, slots=True)
class LoggingCfg(SlottedDefault):
    wandb: Optional[LoggingWandbCfg] = None


def activate_wandb(cfg: object) -> None:
    """Create the wandb run on rank 0 the first time it is called (no-op without a wandb config)."""
    lc = getattr(cfg, "logging", None)
    if logging.wandb is not None or lc is None or lc.wandb is None or distributed.rank != 0:
        return
    try:
        import wandb  # type: ignore
    except ImportError:
        logging.stdout.warning("wandb is not installed; tracking disabled")
        lc.wandb = None
        return
    w = lc.wandb
    run = wandb.init(entity=w.entity, project=w.project, name=w.name, group=w.group,
                     dir=os.environ.get("WANDB_DIR", str(Path.cwd())),
                     config=cfg.to_json_dict() if hasattr(cfg, "to_json_dict") else None)
    for m in METRICS:
        wandb.define_metric(m, step_metric="train/step")
    logging.wandb = run


def setup_logging(cfg: object = None) -> None:
    logging.stdout = StdoutLogger()
