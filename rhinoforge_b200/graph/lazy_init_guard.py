"""Install-completeness guard: state that a captured forward depends on has to exist before the first forward.

A module that creates a buffer, a handle or a cache the first time its ``forward`` runs (``if not hasattr(self, "_rpu_x")``)
is a hazard for every replay mechanism: under stream capture the first call allocates inside the capture and the later
ones take another branch than the recorded one, and a tracing front-end bakes the attribute test into a guard and
recompiles on the second call.  Modules therefore opt into a check at install time: they set a marker and list the
attributes their forward relies on, and :func:`verify_lazy_init` - called at the end of an install and available to
integrators who install by hand - fails if one is missing.  Reference behaviour and names:
``python/rpu_backend/graph/lazy_init_guard.py:23-117``.

Opting in::

    mark_install_checked(module, ("_rpu_engine", "_rpu_cos_sin"))    # or set the two attributes yourself
    verify_lazy_init(model)                                           # walks model.modules()

``_rpu_lazy_init_checked`` is the marker; ``_rpu_dynamo_safe`` is accepted as an older spelling of it.
"""
from __future__ import annotations

from typing import Any, Iterable, List, Sequence, Tuple

import torch.nn as nn

MARKERS: Tuple[str, ...] = ("_rpu_lazy_init_checked", "_rpu_dynamo_safe")
REQUIRED_ATTRS = "_rpu_required_attrs"


class UninitializedLazyStateError(RuntimeError):
    """A module that opted into the install check lacks state it declared as required."""


def mark_install_checked(module: Any, required_attrs: Iterable[str] = ()) -> Any:
    """Opt ``module`` into the check; ``required_attrs`` extend what it already declares."""
    have = tuple(getattr(module, REQUIRED_ATTRS, ()))
    extra = tuple(a for a in required_attrs if a not in have)
    setattr(module, REQUIRED_ATTRS, have + extra)
    setattr(module, MARKERS[0], True)
    return module


def _opted_in(module: Any) -> bool:
    return any(bool(getattr(module, m, False)) for m in MARKERS)


def missing_state(model: Any) -> List[Tuple[str, str, List[str]]]:
    """``[(qualified name, class name, missing attributes)]`` over every opted-in sub-module of ``model`` (an object
    that is not an ``nn.Module`` - a runtime handle, say - is checked by itself)."""
    found = []
    members = model.named_modules() if isinstance(model, nn.Module) else [("", model)]
    for name, sub in members:
        if not _opted_in(sub):
            continue
        absent = [a for a in getattr(sub, REQUIRED_ATTRS, ()) if not hasattr(sub, a)]
        if absent:
            found.append((name or "<root>", type(sub).__name__, absent))
    return found


def verify_lazy_init(model: Any) -> None:
    """Raise :class:`UninitializedLazyStateError` listing every opted-in sub-module with missing declared state."""
    problems = missing_state(model)
    if not problems:
        return
    lines = "\n".join(f"  {path} ({cls}): missing {absent}" for path, cls, absent in problems)
    raise UninitializedLazyStateError(
        "module state is created lazily inside forward; create it while installing (patch_*_for_rpu() / to_rpu()), "
        "before anything captures or traces the forward - a first call that allocates takes a different path from "
        f"every later call, so a recorded graph or a traced guard never matches again:\n{lines}")


def verify_graph_module_best_effort(gm: Any, example_inputs: Sequence[Any] = ()) -> None:
    """Check the direct children of a traced graph module (anything with ``_modules``).  Modules reachable only through
    a closure are invisible here, hence best effort; ``example_inputs`` is accepted for signature compatibility."""
    children = getattr(gm, "_modules", None) or {}
    done = set()
    for child in children.values():
        if child is None or id(child) in done:
            continue
        done.add(id(child))
        verify_lazy_init(child)


# spellings kept for code written against the reference
DynamoUnsafeLazyStateError = UninitializedLazyStateError
freeze_for_dynamo = verify_lazy_init
_verify_lazy_init = verify_lazy_init
_verify_lazy_init_best_effort = verify_graph_module_best_effort

__all__ = ["UninitializedLazyStateError", "DynamoUnsafeLazyStateError", "verify_lazy_init", "freeze_for_dynamo",
           "mark_install_checked", "missing_state", "verify_graph_module_best_effort", "MARKERS"]
