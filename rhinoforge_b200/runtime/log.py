"""Verbosity control: six levels shared by the Python logger ``rpu_backend`` and the environment
variable ``RPU_LOG_LEVEL`` (0 SILENT, 1 ERROR, 2 WARN, 3 INFO (default), 4 DEBUG, 5 TRACE).
Reference: ``python/rpu_backend/runtime/log.py:1-112``."""
from __future__ import annotations

import logging
import os

TRACE = 5
logging.addLevelName(TRACE, "TRACE")

_TO_LOGGING = {0: logging.CRITICAL + 1, 1: logging.ERROR, 2: logging.WARNING, 3: logging.INFO, 4: logging.DEBUG,
               5: TRACE}
_LOG = logging.getLogger("rpu_backend")
if not _LOG.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(logging.Formatter("[%(levelname)s] %(message)s"))
    _LOG.addHandler(_h)
_LOG.propagate = False
_level = 3


def set_debug_level(level: int) -> None:
    global _level
    if not (isinstance(level, int) and 0 <= level <= 5):
        raise ValueError(f"level must be in [0, 5], got {level}")
    _level = level
    _LOG.setLevel(_TO_LOGGING[level])


def get_debug_level() -> int:
    return _level


def trace(msg, *args, **kw) -> None:
    _LOG.log(TRACE, msg, *args, **kw)


def _initial_level() -> int:
    raw = os.environ.get("RPU_LOG_LEVEL")
    if raw is None:
        return 3
    try:
        v = int(raw.strip())
    except ValueError:
        return 3
    return v if 0 <= v <= 5 else 3


set_debug_level(_initial_level())

__all__ = ["TRACE", "set_debug_level", "get_debug_level", "trace"]
