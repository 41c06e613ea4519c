"""Validator of per-instance ``_rpu_*`` attributes (reference: ``python/rpu_backend/runtime/hw_attrs.py:25-47,255-460``).

Three classes of attribute exist on a model handle: *public* ones a user may read and write at any time, *cold*
ones that are read once at install / graph BUILD and may not change afterwards, and *internal* ones owned by the
runtime.  ``guard(obj)`` installs a ``__setattr__`` hook that enforces this; writes to unknown ``_rpu_*`` names are
rejected so that a typo cannot silently do nothing."""
from __future__ import annotations

from typing import Any

from .errors import RPUConfigError

PUBLIC = frozenset({"_rpu_last_execution_plan", "_rpu_debug_tag"})
COLD = frozenset({"_rpu_execution", "_rpu_dtype", "_rpu_tp_world", "_rpu_max_seq_len", "_rpu_chunk_envelope",
                  "_rpu_vlm_chunk_size", "_rpu_linear_partition"})
INTERNAL = frozenset({"_rpu_is_ready", "_rpu_handle", "_rpu_graph_caches", "_rpu_swizzle_started", "_rpu_frozen",
                      # the install-completeness guard's opt-in marker (two spellings) and its attribute list
                      "_rpu_lazy_init_checked", "_rpu_dynamo_safe", "_rpu_required_attrs"})


def classify(name: str) -> str:
    if name in PUBLIC:
        return "public"
    if name in COLD:
        return "cold"
    if name in INTERNAL:
        return "internal"
    return "unknown" if name.startswith("_rpu_") else "foreign"


def validate_write(obj: Any, name: str, value: Any, *, frozen: bool, internal_ok: bool = False) -> None:
    kind = classify(name)
    if kind in ("foreign", "public"):
        return
    if kind == "unknown":
        raise RPUConfigError(f"{name!r} is not a known runtime attribute (known: {sorted(PUBLIC | COLD)})")
    if kind == "internal" and not internal_ok:
        raise RPUConfigError(f"{name!r} is owned by the runtime and cannot be set")
    if kind == "cold" and frozen and getattr(obj, name, value) != value:
        raise RPUConfigError(f"{name!r} is read at install / graph BUILD; it cannot change afterwards "
                             f"(current {getattr(obj, name)!r}, new {value!r})")


def guard(cls):
    """Class decorator: instances validate ``_rpu_*`` writes; ``obj._rpu_freeze()`` starts the cold period."""
    orig = cls.__setattr__

    def __setattr__(self, name, value):
        if name.startswith("_rpu_") and name != "_rpu_frozen":
            validate_write(self, name, value, frozen=self.__dict__.get("_rpu_frozen", False),
                           internal_ok=not self.__dict__.get("_rpu_frozen", False))
        orig(self, name, value)

    def _rpu_freeze(self):
        orig(self, "_rpu_frozen", True)

    cls.__setattr__ = __setattr__
    cls._rpu_freeze = _rpu_freeze
    return cls


__all__ = ["PUBLIC", "COLD", "INTERNAL", "classify", "validate_write", "guard"]
