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


# ---------------------------------------------------------------------------------------------- whole-tree API
# The same policy applied to an object tree that this package does not own (a Hugging Face module tree an integrator
# installs by hand): scans before and after the install, then a per-instance stamp that routes later ``_rpu_*`` writes
# through ``validate_write``.  Reference counterpart: ``python/rpu_backend/runtime/hw_attrs.py:334-472``.
import weakref

USER_SETTABLE_BEFORE_INSTALL = PUBLIC | frozenset({"_rpu_execution", "_rpu_max_seq_len", "_rpu_chunk_envelope",
                                                   "_rpu_vlm_chunk_size"})


class TreeState:
    """Shared by every stamped member of one tree: flipping it on the root is seen by all of them."""

    __slots__ = ("first_forward_done", "__weakref__")

    def __init__(self) -> None:
        self.first_forward_done = False


_STATE_OF: "weakref.WeakKeyDictionary[Any, TreeState]" = weakref.WeakKeyDictionary()
_STAMPED_CLASS: dict = {}


def _members(root: Any):
    walk = getattr(root, "modules", None)
    return list(walk()) if callable(walk) else [root]


def _own_rpu_names(obj: Any):
    return [n for n in list(vars(obj)) if n.startswith("_rpu_")] if hasattr(obj, "__dict__") else []


def validate_preinstall(root: Any) -> None:
    """Before an install: only names a user may set ahead of time can be present; anything the runtime owns is stale
    state from an earlier install and is refused."""
    for m in _members(root):
        for name in _own_rpu_names(m):
            if name not in USER_SETTABLE_BEFORE_INSTALL:
                raise RPUConfigError(f"unexpected attribute {name!r} on {type(m).__name__} before the install; only "
                                     f"{sorted(USER_SETTABLE_BEFORE_INSTALL)} may be set ahead of it - clear the stale "
                                     "state or load a fresh model instance")


def validate_postinstall(root: Any) -> None:
    """After an install: every ``_rpu_*`` name in the tree must be a known one (a typo must not silently do nothing)."""
    for m in _members(root):
        for name in _own_rpu_names(m):
            if classify(name) == "unknown":
                raise RPUConfigError(f"unexpected attribute {name!r} on {type(m).__name__} after the install "
                                     f"(known: {sorted(PUBLIC | COLD | INTERNAL)})")


validate_existing_hw_attrs = validate_postinstall


def _stamped(cls: type) -> type:
    hit = _STAMPED_CLASS.get(cls)
    if hit is None:
        def __setattr__(self, name, value, _base=cls):
            if name.startswith("_rpu_"):
                st = _STATE_OF.get(self)
                frozen = bool(st and st.first_forward_done)
                validate_write(self, name, value, frozen=frozen, internal_ok=not frozen)
            _base.__setattr__(self, name, value)
        hit = type(f"Validated_{cls.__name__}", (cls,), {"__setattr__": __setattr__, "__module__": cls.__module__,
                                                         "_rpu_validated_base": cls})
        _STAMPED_CLASS[cls] = hit
    return hit


def install_hw_attr_validator(root: Any) -> None:
    """Stamp every member of the tree (idempotent): later ``_rpu_*`` writes are checked, and after
    :func:`mark_first_forward_done` cold names cannot change and runtime-owned names cannot be written.  The tree is
    scanned before anything is stamped, so a failure leaves it untouched."""
    validate_postinstall(root)
    if root in _STATE_OF:
        return
    members = _members(root)
    state = TreeState()
    for m in members:
        base = type(m)
        if getattr(base, "_rpu_validated_base", None) is None:
            try:
                m.__class__ = _stamped(base)
            except TypeError as e:
                raise RPUConfigError(f"{base.__name__} does not allow the validator to be installed: {e}") from None
        _STATE_OF[m] = state


def mark_first_forward_done(root: Any) -> None:
    """Start the cold period of a stamped tree; a no-op for objects that were never stamped."""
    try:
        st = _STATE_OF.get(root)
    except TypeError:
        return
    if st is not None:
        st.first_forward_done = True


__all__ = ["PUBLIC", "COLD", "INTERNAL", "classify", "validate_write", "guard", "validate_preinstall",
           "validate_postinstall", "validate_existing_hw_attrs", "install_hw_attr_validator", "mark_first_forward_done",
           "USER_SETTABLE_BEFORE_INSTALL", "TreeState"]
