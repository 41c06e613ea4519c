"""``RhinoVLAPolicy``: one lifecycle for RhinoVLA runtimes that are assembled outside this package.

The RhinoVLA model repository decides how a checkpoint is composed, how requests are pre-processed and what a live
request contains; this package supplies the components such a runtime is built from.  The policy object therefore does
not load anything itself.  It takes a finished runtime (``from_runtime``), or a factory that makes one (``from_factory``,
``from_pretrained``; a callable or a ``"module:callable"`` string), and gives integrators three stable calls -
``prepare_graphs``, ``predict`` and ``predict_action_chunk`` - plus a check that the runtime really executed with the
``rpu_execution`` configuration the caller asked for.  Contract as in the reference,
``python/rpu_backend/api/rhinovla.py:24-450``.

The execution handshake, when the caller passes a non-empty ``rpu_execution``:

* the factory and the runtime each declare ``_rpu_execution_capabilities = {stage: (field, ...)}``; a requested stage or
  field outside that declaration is refused before the factory runs;
* the runtime exposes the configuration it adopted as ``_rpu_execution``; a value that differs from the request is a
  conflict, a missing one means the request was silently dropped and is refused as well;
* every ``prepare_graphs`` / ``predict`` has to bump ``_rpu_execution_resolved_generation`` and publish
  ``_rpu_execution_resolved = {stage: {logical_len, execution_len, chunk_size, padding_rows[, execution_alignment]}}``;
  the numbers are checked for internal consistency and against the exact values and budgets of the request, and the
  checked plan is kept in ``last_rpu_execution_plan``.
"""
from __future__ import annotations

import importlib
import os
from collections.abc import Callable, Collection, Mapping
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple, Union

from ._execution import FIELDS, STAGES, normalize_rpu_execution

RuntimeFactory = Union[str, Callable[..., Any]]
_ABSENT = object()
_PLAN_REQUIRED = ("logical_len", "execution_len", "chunk_size", "padding_rows")
_PLAN_OPTIONAL = ("execution_alignment",)
_ROW_QUANTUM = 16            # a chunk is a whole number of 16-row MMA slabs


def _plain_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def declared_capabilities(owner: Any, where: str) -> Dict[str, Tuple[str, ...]]:
    """``owner._rpu_execution_capabilities`` as ``{stage: fields in canonical order}``; raises when it is missing or
    names a stage or field that does not exist."""
    raw = getattr(owner, "_rpu_execution_capabilities", _ABSENT)
    if raw is _ABSENT:
        raise ValueError(f"{where}: non-empty rpu_execution requires _rpu_execution_capabilities on the runtime "
                         "factory and returned runtime")
    if not isinstance(raw, Mapping):
        raise TypeError(f"{where}: _rpu_execution_capabilities must be a mapping")
    stray = [s for s in raw if s not in STAGES]
    if stray:
        raise ValueError(f"{where}: capability has unknown stage(s) {sorted(map(str, stray))}")
    out: Dict[str, Tuple[str, ...]] = {}
    for stage, fields in raw.items():
        if isinstance(fields, (str, bytes)) or not isinstance(fields, Collection):
            raise TypeError(f"{where}: capability for {stage!r} must be a collection of field names")
        stray_f = [f for f in fields if f not in FIELDS]
        if stray_f:
            raise ValueError(f"{where}: capability for {stage!r} has unknown field(s) {sorted(map(str, stray_f))}")
        out[stage] = tuple(f for f in FIELDS if f in fields)
    return out


def _generation(runtime: Any, where: str) -> int:
    g = getattr(runtime, "_rpu_execution_resolved_generation", _ABSENT)
    if g is _ABSENT:
        return -1
    if not _plain_int(g) or g < 0:
        raise TypeError(f"{where}: _rpu_execution_resolved_generation must be a non-negative integer")
    return g


@dataclass(frozen=True)
class StagePlan:
    """What one stage actually ran with, as published by the runtime after a dispatch."""

    logical_len: int
    execution_len: int
    chunk_size: int
    padding_rows: int
    execution_alignment: Optional[int] = None

    @classmethod
    def parse(cls, stage: str, raw: Any, where: str) -> "StagePlan":
        if not isinstance(raw, Mapping):
            raise RuntimeError(f"{where}: resolved plan is missing stage {stage!r}")
        missing = sorted(set(_PLAN_REQUIRED) - set(raw))
        unknown = sorted(map(str, set(raw) - set(_PLAN_REQUIRED) - set(_PLAN_OPTIONAL)))
        if missing or unknown:
            raise RuntimeError(f"{where}: resolved {stage!r} plan has missing={missing} unknown={unknown}")
        vals = {k: raw[k] for k in (*_PLAN_REQUIRED, *_PLAN_OPTIONAL) if k in raw}
        if not all(_plain_int(v) for v in vals.values()):
            raise TypeError(f"{where}: resolved {stage!r} plan values must be integers")
        plan = cls(**vals)
        if not plan.consistent():
            raise RuntimeError(f"{where}: invalid resolved {stage!r} plan {plan.as_dict()}")
        return plan

    @property
    def alignment(self) -> int:
        return 1 if self.execution_alignment is None else self.execution_alignment

    def consistent(self) -> bool:
        """Lengths add up, the executed length honours its alignment, the chunk is a positive multiple of 16."""
        return (self.logical_len >= 0 and self.padding_rows >= 0
                and self.execution_len == self.logical_len + self.padding_rows
                and self.alignment > 0 and self.execution_len % self.alignment == 0
                and self.chunk_size > 0 and self.chunk_size % _ROW_QUANTUM == 0)

    @property
    def mandatory_padding(self) -> int:
        """Rows the alignment forces, whatever the caller's budget says."""
        return (-self.logical_len) % self.alignment

    def honours(self, request: Mapping[str, Any], stage: str, where: str) -> None:
        """Exact requests must be met exactly; ``padding_budget`` bounds only the padding beyond the mandatory part."""
        want_chunk, want_pad, budget = (request.get(k) for k in FIELDS)
        if _plain_int(want_chunk) and self.chunk_size != want_chunk:
            raise RuntimeError(f"{where}: resolved {stage!r} chunk_size={self.chunk_size} does not match exact "
                               f"request {want_chunk}")
        if _plain_int(want_pad) and self.padding_rows != want_pad:
            raise RuntimeError(f"{where}: resolved {stage!r} padding_rows={self.padding_rows} does not match exact "
                               f"request {want_pad}")
        optional = self.padding_rows - self.mandatory_padding
        if _plain_int(budget) and optional > budget:
            raise RuntimeError(f"{where}: resolved {stage!r} optional padding={optional} (total={self.padding_rows}, "
                               f"mandatory={self.mandatory_padding}, alignment={self.alignment}) exceeds budget {budget}")

    def as_dict(self) -> Dict[str, int]:
        d = {k: getattr(self, k) for k in _PLAN_REQUIRED}
        if self.execution_alignment is not None:
            d["execution_alignment"] = self.execution_alignment
        return d


def check_resolved_execution(runtime: Any, requested: Mapping[str, Mapping[str, Any]], *, previous_generation: int,
                             where: str) -> Dict[str, Dict[str, int]]:
    """Read what the runtime published during the dispatch that just ended and hold it against ``requested``."""
    if _generation(runtime, where) <= previous_generation:
        raise RuntimeError(f"{where}: runtime did not publish a fresh resolved execution plan; "
                           "_rpu_execution_resolved_generation must strictly increase during this dispatch")
    published = getattr(runtime, "_rpu_execution_resolved", _ABSENT)
    if published is _ABSENT:
        raise RuntimeError(f"{where}: runtime did not publish _rpu_execution_resolved after execution")
    if not isinstance(published, Mapping):
        raise TypeError(f"{where}: _rpu_execution_resolved must be a mapping")
    checked: Dict[str, Dict[str, int]] = {}
    for stage, request in requested.items():
        plan = StagePlan.parse(stage, published.get(stage), where)
        plan.honours(request, stage, where)
        checked[stage] = plan.as_dict()
    return checked


def resolve_runtime_factory(target: RuntimeFactory) -> Callable[..., Any]:
    """A callable is returned as is; ``"package.module:name"`` is imported and looked up."""
    if callable(target):
        return target
    if not isinstance(target, str):
        raise TypeError(f"RhinoVLA runtime_factory must be callable or 'module:callable', got {type(target).__name__}")
    module, colon, name = target.partition(":")
    if not (colon and module and name):
        raise ValueError(f"RhinoVLA runtime_factory must use 'module:callable' syntax, got {target!r}")
    found = getattr(importlib.import_module(module), name)
    if not callable(found):
        raise TypeError(f"RhinoVLA runtime factory is not callable: {target}")
    return found


def _negotiate(rpu_execution: Any, owner: Any, where: str) -> Mapping:
    """Normalise a request and, if it asks for anything, restrict it to what ``owner`` declares."""
    cfg = normalize_rpu_execution(rpu_execution, entry_point=where)
    if cfg:
        cfg = normalize_rpu_execution(cfg, entry_point=where, supported=declared_capabilities(owner, where))
    return cfg


class _Dispatch:
    """Brackets one runtime call: remembers the plan generation before it, validates the published plan after it."""

    def __init__(self, policy: "RhinoVLAPolicy", where: str):
        self.policy, self.where = policy, where
        self.before = -1

    def __enter__(self) -> "_Dispatch":
        if self.policy._rpu_execution_handshake_required:
            self.before = _generation(self.policy._runtime, self.where)
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        p = self.policy
        if exc_type is None and p._rpu_execution_handshake_required:
            p._last_rpu_execution_plan = check_resolved_execution(p._runtime, p._rpu_execution,
                                                                  previous_generation=self.before, where=self.where)
        return False


class RhinoVLAPolicy:
    """Policy facade over a runtime that the RhinoVLA model repository assembled."""

    FAMILY = "RhinoVLA"

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        raise RuntimeError("RhinoVLAPolicy() is not a public constructor. Use from_runtime(), from_factory(), or "
                           "from_pretrained().")

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_runtime(cls, runtime: Any, *, rpu_execution: Optional[Mapping] = None) -> "RhinoVLAPolicy":
        """Wrap an assembled runtime (anything with ``predict(**request)``).  Passing a policy returns that policy,
        after checking that ``rpu_execution`` - if given - equals what it already holds."""
        where = "RhinoVLAPolicy.from_runtime"
        if isinstance(runtime, cls):
            return cls._rewrap(runtime, rpu_execution, where)
        if not callable(getattr(runtime, "predict", None)):
            raise TypeError("RhinoVLA runtime must provide callable predict(**request)")
        adopted = getattr(runtime, "_rpu_execution", _ABSENT)
        asked = rpu_execution is not None
        cfg = _negotiate(rpu_execution if asked else (None if adopted is _ABSENT else adopted), runtime, where)
        if adopted is _ABSENT:
            if asked and cfg:
                raise ValueError(f"{where}: non-empty rpu_execution was not consumed by the runtime; the runtime must "
                                 "expose its effective configuration as _rpu_execution")
        else:
            effective = normalize_rpu_execution(adopted, entry_point=where)
            if asked and cfg != effective:
                raise ValueError(f"{where}: rpu_execution conflicts with the runtime's effective configuration")
            cfg = effective
        self = cls.__new__(cls)
        self._runtime = runtime
        self._rpu_execution = cfg
        self._rpu_execution_handshake_required = asked and bool(cfg)
        self._last_rpu_execution_plan = {}
        return self

    @classmethod
    def _rewrap(cls, policy: "RhinoVLAPolicy", rpu_execution: Optional[Mapping], where: str) -> "RhinoVLAPolicy":
        if rpu_execution is None:
            return policy
        cfg = _negotiate(rpu_execution, policy._runtime, where)
        if cfg != normalize_rpu_execution(getattr(policy, "_rpu_execution", None), entry_point=where):
            raise ValueError(f"{where}: rpu_execution conflicts with the existing policy configuration")
        policy._rpu_execution_handshake_required = bool(cfg)
        return policy

    @classmethod
    def from_factory(cls, runtime_factory: RuntimeFactory, config: Mapping[str, Any], *,
                     rpu_execution: Optional[Mapping] = None) -> "RhinoVLAPolicy":
        """``factory(config)`` - or ``factory(config, rpu_execution=cfg)`` when the caller passed one - makes the
        runtime."""
        where = "RhinoVLAPolicy.from_factory"
        if not isinstance(config, Mapping):
            raise TypeError(f"RhinoVLA factory config must be a mapping, got {type(config).__name__}")
        normalize_rpu_execution(rpu_execution, entry_point=where)          # shape errors before the import
        factory = resolve_runtime_factory(runtime_factory)
        cfg = _negotiate(rpu_execution, factory, where)
        if rpu_execution is None:
            return cls.from_runtime(factory(config))
        return cls.from_runtime(factory(config, rpu_execution=cfg), rpu_execution=cfg)

    @classmethod
    def from_pretrained(cls, pretrained_name_or_path: Union[str, "os.PathLike[str]"], *,
                        runtime_factory: RuntimeFactory, config: Optional[Mapping[str, Any]] = None,
                        rpu_execution: Optional[Mapping] = None, **factory_kwargs: Any) -> "RhinoVLAPolicy":
        """``factory(pretrained_name_or_path, **factory_kwargs)`` makes the runtime; ``config`` and ``rpu_execution``
        travel as keyword arguments when given.  Loading, weight conversion and input validation are the factory's."""
        where = "RhinoVLAPolicy.from_pretrained"
        if isinstance(pretrained_name_or_path, str):
            text = pretrained_name_or_path
        elif isinstance(pretrained_name_or_path, os.PathLike):
            text = os.fspath(pretrained_name_or_path)
            if not isinstance(text, str):
                raise TypeError("RhinoVLA pretrained_name_or_path PathLike must resolve to str")
        else:
            raise TypeError("RhinoVLA pretrained_name_or_path must be str or PathLike, got "
                            f"{type(pretrained_name_or_path).__name__}")
        if not text:
            raise ValueError("RhinoVLA pretrained_name_or_path must not be empty")
        normalize_rpu_execution(rpu_execution, entry_point=where)
        factory = resolve_runtime_factory(runtime_factory)
        cfg = _negotiate(rpu_execution, factory, where)
        if config is not None:
            if not isinstance(config, Mapping):
                raise TypeError(f"RhinoVLA config must be a mapping, got {type(config).__name__}")
            factory_kwargs["config"] = config
        if rpu_execution is not None:
            factory_kwargs["rpu_execution"] = cfg
        runtime = factory(pretrained_name_or_path, **factory_kwargs)
        return cls.from_runtime(runtime, rpu_execution=cfg if rpu_execution is not None else None)

    # ------------------------------------------------------------------ use
    @property
    def runtime(self) -> Any:
        """The wrapped runtime (model-specific diagnostics live there)."""
        return self._runtime

    @property
    def rpu_execution(self) -> Mapping:
        """The frozen execution configuration in force."""
        return self._rpu_execution

    @property
    def last_rpu_execution_plan(self) -> Dict[str, Dict[str, int]]:
        """A detached copy of the per-stage plan validated after the last dispatch (empty without a handshake)."""
        return {stage: dict(plan) for stage, plan in self._last_rpu_execution_plan.items()}

    def prepare_graphs(self, **request: Any) -> Any:
        """Have the runtime build its finite set of graphs for a representative request."""
        prepare = getattr(self._runtime, "prepare_graphs", None)
        if not callable(prepare):
            raise TypeError("RhinoVLA runtime does not provide prepare_graphs(**request)")
        with _Dispatch(self, "RhinoVLAPolicy.prepare_graphs"):
            return prepare(**request)

    def predict(self, **request: Any) -> Any:
        """One complete request -> its action chunk."""
        with _Dispatch(self, "RhinoVLAPolicy.predict"):
            return self._runtime.predict(**request)

    def predict_action_chunk(self, **request: Any) -> Any:
        """The VLA-policy spelling of :meth:`predict`."""
        return self.predict(**request)


__all__ = ["RhinoVLAPolicy", "StagePlan", "check_resolved_execution", "declared_capabilities",
           "resolve_runtime_factory"]
