"""Configuration base class.

Every ``*Cfg`` in the framework is a ``@dataclass(init=False, slots=True)`` deriving from
:class:`SlottedDefault`: constructing it with no arguments fills every field that declares a
default and leaves required fields unset, so a user script assigns exactly what it cares about and
a missing required field surfaces as ``AttributeError`` at first use. Same contract as
pithtrain/config.py:9-48 of the reference.
"""

from __future__ import annotations

from dataclasses import MISSING, fields, is_dataclass
from datetime import timedelta
from functools import partial
from pathlib import Path
from typing import Any


class SlottedDefault:
    __slots__ = ()

    def __init__(self) -> None:
        for f in fields(self):  # type: ignore[arg-type]
            if f.default is not MISSING:
                setattr(self, f.name, f.default)
            elif f.default_factory is not MISSING:  # type: ignore[misc]
                setattr(self, f.name, f.default_factory())  # type: ignore[misc]

    def to_json_dict(self) -> dict:
        """JSON-serialisable view (unset required fields are skipped)."""
        out: dict[str, Any] = {}
        for f in fields(self):  # type: ignore[arg-type]
            if hasattr(self, f.name):
                out[f.name] = _jsonable(getattr(self, f.name))
        return out


def _jsonable(obj: Any) -> Any:
    if isinstance(obj, SlottedDefault):
        return obj.to_json_dict()
    if is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: _jsonable(getattr(obj, f.name)) for f in fields(obj) if hasattr(obj, f.name)}
    if isinstance(obj, dict):
        return {str(k): _jsonable(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_jsonable(v) for v in obj]
    if isinstance(obj, Path):
        return str(obj)
    if isinstance(obj, timedelta):
        return obj.total_seconds()
    if isinstance(obj, partial):
        name = getattr(obj.func, "__name__", repr(obj.func))
        kw = ", ".join(f"{k}={v!r}" for k, v in obj.keywords.items())
        return f"{name}({kw})" if kw else name
    if callable(obj):
        return getattr(obj, "__name__", repr(obj))
    return obj
