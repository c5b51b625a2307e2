"""Runtime state of logging, populated by :func:`pithtrain_b200.modules.logging.setup_logging`.

``stdout`` is the rank-filtered console logger every module writes step lines and notices through;
``wandb`` is the Weights & Biases run object once tracking has been activated (after the first good
step), ``None`` before that and whenever tracking is not configured.
"""

from __future__ import annotations

from typing import Any, Optional

__all__ = ["stdout", "wandb"]

wandb: Optional[Any] = None
stdout: Any = None
