"""Adapter registry: HF architecture string -> adapter class.

``register_adapter / get_adapter / list_adapters`` are the stable API.  Built-in adapters are
recorded as (module, class) targets and imported only when their architecture is first looked
up; external packages register through the ``rpu_backend.plugins`` entry-point group and can
never replace a built-in.  Behaviour follows ``python/rpu_backend/runtime/registry.py:33-208``.
"""
from __future__ import annotations

import importlib
import importlib.metadata
import threading
import warnings
from dataclasses import dataclass
from types import SimpleNamespace
from typing import Any, Dict, Iterable, List, Tuple

from .errors import UnsupportedModelError

PLUGIN_GROUP = "rpu_backend.plugins"


@dataclass(frozen=True)
class LazyTarget:
    module: str
    attr: str


ADAPTERS: Dict[str, Any] = {}
_lock = threading.RLock()
_plugins_loaded = False


def register_adapter(arch: str, adapter_cls) -> None:
    """Bind ``arch`` to ``adapter_cls``.  Re-registering the same pair is a no-op; a different
    class for a taken architecture raises ``RuntimeError``."""
    with _lock:
        cur = ADAPTERS.get(arch)
        if isinstance(cur, LazyTarget):
            got = (adapter_cls.__module__, adapter_cls.__name__)
            if got != (cur.module, cur.attr):
                raise RuntimeError(f"Adapter already registered for {arch!r}: lazy target "
                                   f"{(cur.module, cur.attr)!r} != {got!r}")
        elif cur is not None and cur is not adapter_cls:
            raise RuntimeError(f"Adapter already registered for {arch!r}: {cur!r} != {adapter_cls!r}")
        ADAPTERS[arch] = adapter_cls


def list_adapters() -> List[str]:
    with _lock:
        return list(ADAPTERS)


def get_adapter(arch: str):
    """Adapter class for ``arch`` (importing a lazy built-in on first use) or ``UnsupportedModelError``."""
    with _lock:
        found = ADAPTERS.get(arch)
    if found is None:
        _load_plugins_once()
    with _lock:
        found = ADAPTERS.get(arch)
        if found is None:
            raise UnsupportedModelError(
                f"No RPU adapter registered for HF architecture {arch!r}. Registered archs: {sorted(ADAPTERS)}.")
        if not isinstance(found, LazyTarget):
            return found
        cls = getattr(importlib.import_module(found.module), found.attr)
        if isinstance(ADAPTERS.get(arch), LazyTarget):
            ADAPTERS[arch] = cls
        if ADAPTERS[arch] is not cls:
            raise RuntimeError(f"Adapter target changed while loading {arch!r}")
        return cls


def register_builtins(builtins: Iterable[Tuple[str, str, str]]) -> None:
    """Record ``(arch, module, class)`` targets without importing anything."""
    with _lock:
        for arch, module, attr in builtins:
            target = LazyTarget(module, attr)
            cur = ADAPTERS.get(arch)
            if cur is None:
                ADAPTERS[arch] = target
            elif cur != target and (getattr(cur, "__module__", None), getattr(cur, "__name__", None)) != (module, attr):
                raise RuntimeError(f"Built-in adapter collision for {arch!r}: {cur!r} != {(module, attr)!r}")


def _plugin_api(builtin_names: frozenset) -> SimpleNamespace:
    def register_plugin_adapter(arch: str, cls) -> None:
        if arch in builtin_names:
            raise RuntimeError(f"{arch} is a built-in; plugins cannot override.")
        register_adapter(arch, cls)
    return SimpleNamespace(register_adapter=register_plugin_adapter)


def discover_entry_points() -> None:
    """Load every ``rpu_backend.plugins`` entry point.  A collision with a built-in propagates;
    any other plugin failure becomes an ``ImportWarning``."""
    global _plugins_loaded
    with _lock:
        api = _plugin_api(frozenset(ADAPTERS))
        for ep in importlib.metadata.entry_points(group=PLUGIN_GROUP):
            try:
                ep.load()(api)
            except RuntimeError:
                raise
            except Exception as e:  # noqa: BLE001
                warnings.warn(f"Entry-point plugin {ep.name!r} failed to register ({type(e).__name__}: {e}). "
                              "Skipping.", ImportWarning, stacklevel=2)
        _plugins_loaded = True


def _load_plugins_once() -> None:
    with _lock:
        if not _plugins_loaded:
            discover_entry_points()


def discover_in_tree(builtins: Iterable[Tuple[str, str, str]] = ()) -> None:
    register_builtins(builtins)


def discover_all(builtins: Iterable[Tuple[str, str, str]] = ()) -> None:
    """Cold-start bootstrap: built-ins only; plugins wait for an unknown-architecture lookup."""
    register_builtins(builtins)
