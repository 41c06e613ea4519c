"""``rpu_execution``: the cold, per-handle execution configuration.

A mapping ``{stage: {field: value}}`` with stages ``prefill | vision | action`` and fields
``chunk_size`` (``"auto"`` or a positive multiple of 16), ``padding_rows`` (``"auto"`` or >= 0,
exact) and ``padding_budget`` (>= 0, an upper bound; conflicts with an exact ``padding_rows``).
It is validated before any weight is touched, deep-frozen, and bound once to the model instance;
binding a different value later is an error.  Contract and messages follow the reference
(``python/rpu_backend/api/_execution.py:60-241``).

On B200 ``chunk_size`` bounds the rows of one packed prefill launch (activation-arena size and
time-to-first-token control); padding fields are accepted for compatibility -- the varlen kernels
need no padded rows, so they only affect how ``RPUCache`` sizes its head-room.
"""
from __future__ import annotations

from collections.abc import Collection, Mapping
from typing import Any, Dict, Optional

STAGES = ("prefill", "vision", "action")
FIELDS = ("chunk_size", "padding_rows", "padding_budget")
_UNSET = object()


class FrozenConfig(Mapping):
    """Immutable mapping; copy/deepcopy return self, pickling round-trips."""

    __slots__ = ("_pairs",)

    def __init__(self, value: Mapping) -> None:
        object.__setattr__(self, "_pairs", tuple(value.items()))

    def __getitem__(self, key):
        for k, v in self._pairs:
            if k == key:
                return v
        raise KeyError(key)

    def __iter__(self):
        return iter(k for k, _ in self._pairs)

    def __len__(self) -> int:
        return len(self._pairs)

    def __setattr__(self, name, value) -> None:
        raise TypeError("rpu_execution is read-only")

    def __delattr__(self, name) -> None:
        raise TypeError("rpu_execution is read-only")

    def __copy__(self):
        return self

    def __deepcopy__(self, memo):
        memo[id(self)] = self
        return self

    def __reduce__(self):
        return (type(self), (dict(self.items()),))

    def __repr__(self) -> str:
        return f"FrozenConfig({dict(self.items())!r})"


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _check_field(entry_point: str, stage: str, field: str, v):
    where = f"{entry_point}: rpu_execution[{stage!r}][{field!r}]"
    if field == "chunk_size":
        if v == "auto" and isinstance(v, str):
            return "auto"
        if not _is_int(v) or v <= 0 or v % 16:
            raise ValueError(f"{where} must be 'auto' or a positive multiple of 16, got {v!r}")
        return v
    if field == "padding_rows":
        if v == "auto" and isinstance(v, str):
            return "auto"
        if not _is_int(v) or v < 0:
            raise ValueError(f"{where} must be 'auto' or a non-negative integer, got {v!r}")
        return v
    if not _is_int(v) or v < 0:
        raise ValueError(f"{where} must be a non-negative integer, got {v!r}")
    return v


def normalize_rpu_execution(value: Optional[Mapping], *, entry_point: str, vlm_chunk_size: Optional[int] = None,
                            supported: Optional[Mapping[str, Collection[str]]] = None) -> Mapping:
    """Validate ``value`` and return a detached, deeply read-only copy (or raise before loading)."""
    if value is None:
        value = {}
    if not isinstance(value, Mapping):
        raise TypeError(f"{entry_point}: rpu_execution must be a mapping, got {type(value).__name__}")
    unknown = set(value) - set(STAGES)
    if unknown:
        raise ValueError(f"{entry_point}: rpu_execution has unknown stage(s) {sorted(map(str, unknown))}; "
                         f"supported stages are {list(STAGES)}")
    if supported is not None:
        bad = set(value) - set(supported)
        if bad:
            raise ValueError(f"{entry_point}: rpu_execution stage(s) {sorted(map(str, bad))} are not supported by "
                             "this model entry point")
    out: Dict[str, Dict[str, Any]] = {}
    for stage in STAGES:
        if stage not in value:
            continue
        sv = value[stage]
        if not isinstance(sv, Mapping):
            raise TypeError(f"{entry_point}: rpu_execution[{stage!r}] must be a mapping, got {type(sv).__name__}")
        unknown_f = set(sv) - set(FIELDS)
        if unknown_f:
            raise ValueError(f"{entry_point}: rpu_execution[{stage!r}] has unknown field(s) "
                             f"{sorted(map(str, unknown_f))}; supported fields are {list(FIELDS)}")
        if supported is not None:
            bad_f = set(sv) - set(supported[stage])
            if bad_f:
                raise ValueError(f"{entry_point}: rpu_execution[{stage!r}] field(s) {sorted(map(str, bad_f))} are "
                                 "not supported by this model entry point")
        cfg = {f: _check_field(entry_point, stage, f, sv[f]) for f in FIELDS if f in sv}
        if _is_int(cfg.get("padding_rows")) and "padding_budget" in cfg:
            raise ValueError(f"{entry_point}: rpu_execution[{stage!r}]['padding_rows'] is exact and conflicts with "
                             "'padding_budget'")
        if cfg:
            out[stage] = cfg
    if vlm_chunk_size is not None:
        if not _is_int(vlm_chunk_size) or vlm_chunk_size < 0 or (vlm_chunk_size and vlm_chunk_size % 16):
            raise ValueError(f"{entry_point}: vlm_chunk_size must be 0 or a positive multiple of 16, "
                             f"got {vlm_chunk_size!r}")
        if "chunk_size" in out.get("prefill", {}):
            raise ValueError(f"{entry_point}: vlm_chunk_size conflicts with rpu_execution['prefill']['chunk_size']; "
                             "pass only one")
        out.setdefault("prefill", {})["chunk_size"] = "auto" if vlm_chunk_size == 0 else vlm_chunk_size
    return FrozenConfig({s: FrozenConfig({f: out[s][f] for f in FIELDS if f in out[s]}) for s in STAGES if s in out})


def bind_rpu_execution(owner: Any, value: Optional[Mapping] = None, *, entry_point: str,
                       supported: Optional[Mapping[str, Collection[str]]] = None) -> Mapping:
    """Attach one validated config to ``owner._rpu_execution``; an equal existing config is kept,
    a different one is a conflict."""
    existing = getattr(owner, "_rpu_execution", _UNSET)
    wanted = normalize_rpu_execution(existing if (value is None and existing is not _UNSET) else value,
                                     entry_point=entry_point, supported=supported)
    if existing is not _UNSET:
        current = normalize_rpu_execution(existing, entry_point=entry_point, supported=supported)
        if value is not None and current != wanted:
            raise ValueError(f"{entry_point}: rpu_execution conflicts with the existing model configuration")
        if isinstance(existing, FrozenConfig) and all(isinstance(v, FrozenConfig) for v in existing.values()) \
                and existing == current:
            return existing
        wanted = current
    owner._rpu_execution = wanted
    return wanted


def prefill_chunk_rows(cfg: Mapping, stage: str = "prefill", default: int = 8192) -> int:
    """Rows of one packed prefill launch implied by a normalised config."""
    v = cfg.get(stage, {}).get("chunk_size", "auto") if cfg else "auto"
    return default if v == "auto" else int(v)


__all__ = ["bind_rpu_execution", "normalize_rpu_execution", "prefill_chunk_rows", "FrozenConfig", "STAGES", "FIELDS"]
