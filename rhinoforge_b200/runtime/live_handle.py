"""Process-wide single-live-handle gate.

One fused model or policy may be live per process; a second load raises
``RPUSingleHandleError`` until the first owner is garbage-collected.  A failure after the
irreversible weight transform began makes the slot terminal: only a fresh process may load again.
Contract: ``python/rpu_backend/api/causal_lm.py:64-128``.
"""
from __future__ import annotations

import threading
import weakref
from typing import Optional

_lock = threading.RLock()
_ref: Optional[weakref.ref] = None
_alias: Optional[weakref.ref] = None
_terminal: Optional[str] = None


def _release(_r=None) -> None:
    global _ref, _alias
    with _lock:
        live = _ref() if _ref is not None else None
        alt = _alias() if _alias is not None else None
        if live is None and alt is None:
            _ref = None
            _alias = None


def _live():
    a = _ref() if _ref is not None else None
    b = _alias() if _alias is not None else None
    return a if a is not None else b


def claim(owner) -> int:
    from ..api.errors import RPUSingleHandleError
    global _ref
    with _lock:
        live = _live()
        if _terminal is not None:
            if live is owner:
                return id(owner)
            raise RPUSingleHandleError("This process cannot create another RPU model/policy after a process-terminal "
                                       f"owner: {_terminal}. Restart the Python process before loading another one.")
        if live is not None and live is not owner and (_alias is None or _alias() is not owner):
            raise RPUSingleHandleError(
                f"An RPU model/policy is already live in this process (type={type(live).__name__}, id={id(live)}). "
                "Call `del model; import gc; gc.collect()` to release it before loading a new one.")
        _ref = weakref.ref(owner, _release)
        return id(owner)


def rebind(owner, handle) -> None:
    """Keep the slot claimed while either the original owner or its runtime handle is alive."""
    global _alias
    with _lock:
        _alias = weakref.ref(handle, _release)


def release(owner=None) -> None:
    global _ref, _alias
    with _lock:
        if _terminal is None:
            _ref = None
            _alias = None


def poison(owner, reason: str) -> None:
    global _terminal
    with _lock:
        if _terminal is None:
            _terminal = str(reason)


def is_live() -> bool:
    with _lock:
        return _live() is not None


def _reset_for_tests() -> None:
    global _ref, _alias, _terminal
    with _lock:
        _ref = _alias = _terminal = None
