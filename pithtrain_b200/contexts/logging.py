"""Logging runtime state (filled by ``modules.logging.setup_logging``)."""
from typing import Any, Optional

stdout: Any = None
wandb: Optional[Any] = None
