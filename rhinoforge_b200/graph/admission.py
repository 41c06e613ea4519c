"""Graph admission: turning one call into a :class:`GraphSignature`, explaining misses, and a front LRU.

The native cache (``csrc/runtime/graph_exec.cpp``) is the authority on what is captured; this module is the
Python side that both capture front-ends share (reference behaviour: ``python/rpu_backend/graph/admission.py:
244-434,464-601``):

* :class:`SignaturePlanner` walks the arguments of a call and derives the signature *layers* - tensor structure
  (how many tensors, their ranks and where they sit in the argument tree), literal shapes, dtypes + memory
  layout, hashed scalar arguments, a branch key for the callable and a segment key - and from them the
  ``GraphSignature`` the native cache is keyed by.
* :meth:`SignaturePlanner.attribute_miss_reason` names the first layer in which a new call differs from the
  closest known entry (``no_entry``, ``gm_id``, ``tensor_struct``, ``shape_bucket``, ``dtype_layout``,
  ``scalar_flags``, ``branch_key``, ``segment_key``).
* :class:`GraphPlan` records what was decided for one call (record / replay / recapture; retain / evict).
* :class:`EntryRegistry` is a least-recently-used table in front of a ``GraphCache`` that evicts the coldest
  signature when a new one arrives at capacity (never from a frozen cache: a READY cache refuses new entries).
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ._runtime import GraphCache, GraphSignature, fnv1a_64

WORKLOAD_PREFILL, WORKLOAD_DECODE, WORKLOAD_GENERIC = "prefill", "decode", "generic"
WORKLOAD_KINDS = (WORKLOAD_PREFILL, WORKLOAD_DECODE, WORKLOAD_GENERIC)
ADMISSION_RECORD, ADMISSION_REPLAY, ADMISSION_RECAPTURE = "record", "replay", "recapture"
ADMISSION_KINDS = (ADMISSION_RECORD, ADMISSION_REPLAY, ADMISSION_RECAPTURE)
LIFECYCLE_RETAIN, LIFECYCLE_EVICT = "retain", "evict"
MISS_REASONS = ("no_entry", "gm_id", "tensor_struct", "shape_bucket", "dtype_layout", "scalar_flags", "branch_key",
                "segment_key")
_LAYER_ORDER = MISS_REASONS[1:]

_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int8, torch.uint8, torch.int16,
           torch.int32, torch.int64, torch.bool)
_DTYPE_ID = {d: i + 1 for i, d in enumerate(_DTYPES)}


@dataclass(frozen=True)
class SignatureLayers:
    """The comparable pieces of a signature, outermost first."""
    gm_id: int
    tensor_struct: Tuple[int, ...]
    shape_bucket: Tuple[int, ...]
    dtype_layout: Tuple[int, ...]
    scalar_flags: int
    branch_key: int
    segment_key: int

    def first_divergence(self, other: "SignatureLayers") -> Optional[str]:
        for name in _LAYER_ORDER:
            if getattr(self, name) != getattr(other, name):
                return name
        return None


@dataclass
class GraphPlan:
    signature: GraphSignature
    layers: SignatureLayers
    workload: str = WORKLOAD_GENERIC
    admission: str = ADMISSION_RECORD
    lifecycle: str = LIFECYCLE_RETAIN
    miss_reason: Optional[str] = None
    evicted: List[Tuple] = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.workload not in WORKLOAD_KINDS:
            raise ValueError(f"unknown workload kind {self.workload!r}")
        if self.admission not in ADMISSION_KINDS:
            raise ValueError(f"unknown admission kind {self.admission!r}")

    def to_log_str(self) -> str:
        why = f" miss={self.miss_reason}" if self.miss_reason else ""
        return (f"plan[{self.workload}] {self.admission}/{self.lifecycle}{why} shapes={list(self.layers.shape_bucket)} "
                f"branch={self.layers.branch_key:#x} segment={self.layers.segment_key}")


def _scalar_token(v: Any) -> str:
    if isinstance(v, bool):
        return f"b{int(v)}"
    if isinstance(v, int):
        return f"i{v}"
    if isinstance(v, float):
        return f"f{v!r}"
    if isinstance(v, str):
        return f"s{v}"
    if v is None:
        return "n"
    if isinstance(v, (torch.dtype, torch.device)):
        return f"t{v}"
    return f"o{type(v).__module__}.{type(v).__qualname__}"


class SignaturePlanner:
    """Derives signatures from call arguments; stateless apart from an optional debug log."""

    def __init__(self, *, debug: bool = False):
        self.debug = debug
        self.log: List[str] = []

    @staticmethod
    def stable_branch_key(value: Any) -> int:
        """A key that survives process restarts: callables by module + qualified name, everything else by its
        scalar token.  Bound methods include the class of their owner, not its address."""
        if value is None:
            return 0
        if isinstance(value, int) and not isinstance(value, bool):
            return value & 0x7FFFFFFFFFFFFFFF
        if callable(value):
            owner = getattr(value, "__self__", None)
            name = f"{getattr(value, '__module__', '')}.{getattr(value, '__qualname__', type(value).__qualname__)}"
            if owner is not None:
                name = f"{type(owner).__module__}.{type(owner).__qualname__}:{name}"
            return fnv1a_64(name) & 0x7FFFFFFFFFFFFFFF
        return fnv1a_64(_scalar_token(value)) & 0x7FFFFFFFFFFFFFFF

    def _walk(self, obj: Any, path: int, struct: List[int], shapes: List[int], dl: List[int], scalars: List[str]) -> None:
        if isinstance(obj, torch.Tensor):
            struct += [path, obj.dim()]
            shapes += [int(s) for s in obj.shape] or [0]
            layout = (1 if obj.is_contiguous() else 0) | ((1 if obj.is_cuda else 0) << 1)
            dl += [_DTYPE_ID.get(obj.dtype, 0), layout]
        elif isinstance(obj, (list, tuple)):
            struct += [path, -len(obj) - 1]
            for i, v in enumerate(obj):
                self._walk(v, path * 31 + i + 1, struct, shapes, dl, scalars)
        elif isinstance(obj, dict):
            struct += [path, -len(obj) - 1]
            for k in sorted(obj, key=str):
                self._walk(obj[k], path * 31 + (fnv1a_64(str(k)) & 0xFFFF), struct, shapes, dl, scalars)
        else:
            scalars.append(f"{path}:{_scalar_token(obj)}")

    def layers_for_call(self, op_id: Any, args: Sequence[Any] = (), kwargs: Optional[Dict[str, Any]] = None, *,
                        branch: Any = None, segment: int = 0) -> SignatureLayers:
        struct: List[int] = []
        shapes: List[int] = []
        dl: List[int] = []
        scalars: List[str] = []
        self._walk(tuple(args), 1, struct, shapes, dl, scalars)
        if kwargs:
            self._walk(dict(kwargs), 2, struct, shapes, dl, scalars)
        gm = fnv1a_64(op_id) if isinstance(op_id, str) else int(op_id)
        flags = fnv1a_64("|".join(scalars)) & 0x7FFFFFFFFFFFFFFF if scalars else 0
        return SignatureLayers(gm & 0x7FFFFFFFFFFFFFFF, tuple(struct), tuple(shapes), tuple(dl), flags,
                               self.stable_branch_key(branch), int(segment))

    def build_signature(self, op_id: Any, args: Sequence[Any] = (), kwargs: Optional[Dict[str, Any]] = None, *,
                        branch: Any = None, segment: int = 0, dyn_dims: Sequence[int] = ()) -> Tuple[GraphSignature, SignatureLayers]:
        L = self.layers_for_call(op_id, args, kwargs, branch=branch, segment=segment)
        # the native key carries shapes and dtypes literally; structure and layout ride in the flag word
        flags = fnv1a_64(f"{L.scalar_flags}|{L.tensor_struct}|{L.dtype_layout[1::2]}") & 0x7FFFFFFFFFFFFFFF
        sig = GraphSignature(op_id if isinstance(op_id, str) else L.gm_id, L.shape_bucket, tuple(dyn_dims),
                             L.dtype_layout[0::2], flags, L.branch_key, L.segment_key)
        if self.debug:
            self.log.append(f"sig {op_id}: shapes={L.shape_bucket} flags={flags:#x}")
        return sig, L

    @staticmethod
    def infer_workload_kind(args: Sequence[Any], kwargs: Optional[Dict[str, Any]] = None) -> str:
        """``decode`` when the first ``[batch, seq, ...]`` tensor has one row per sequence, ``prefill`` when it has
        more, ``generic`` when no such tensor is passed."""
        stack = list(args) + list((kwargs or {}).values())
        while stack:
            v = stack.pop(0)
            if isinstance(v, torch.Tensor) and v.dim() >= 2:
                return WORKLOAD_DECODE if v.shape[1] == 1 else WORKLOAD_PREFILL
            if isinstance(v, (list, tuple)):
                stack = list(v) + stack
        return WORKLOAD_GENERIC

    @staticmethod
    def attribute_miss_reason(new: SignatureLayers, known: Sequence[SignatureLayers]) -> str:
        """The outermost layer in which ``new`` differs from its closest known entry (the entry that agrees on the
        most leading layers); ``no_entry`` for an empty table."""
        if not known:
            return "no_entry"
        best_depth, best = -1, "gm_id"
        for k in known:
            d = new.first_divergence(k)
            if d is None:
                return "no_entry"          # an identical entry exists: the miss is not a signature miss
            depth = _LAYER_ORDER.index(d)
            if depth > best_depth:
                best_depth, best = depth, d
        return best


class EntryRegistry:
    """Front LRU over one ``GraphCache``: admits a plan, evicting the coldest signature at capacity."""

    def __init__(self, cache: Optional[GraphCache] = None, *, max_entries: int = GraphCache.DEFAULT_MAX_ENTRIES,
                 planner: Optional[SignaturePlanner] = None):
        if max_entries < 1:
            raise ValueError("max_entries must be positive")
        self._cache = cache if cache is not None else GraphCache(max_entries)
        self._planner = planner or SignaturePlanner()
        self._max = int(max_entries)
        self._lru: "OrderedDict[GraphSignature, SignatureLayers]" = OrderedDict()
        self._evict_total = 0
        self._hits = 0
        self._misses = 0
        self._miss_reasons: Dict[str, int] = {}

    @property
    def cache(self) -> GraphCache:
        return self._cache

    @property
    def planner(self) -> SignaturePlanner:
        return self._planner

    @property
    def evict_total(self) -> int:
        return self._evict_total

    def plan_for_call(self, op_id: Any, args: Sequence[Any] = (), kwargs: Optional[Dict[str, Any]] = None, *,
                      branch: Any = None, segment: int = 0) -> GraphPlan:
        sig, layers = self._planner.build_signature(op_id, args, kwargs, branch=branch, segment=segment)
        plan = GraphPlan(sig, layers, workload=self._planner.infer_workload_kind(args, kwargs))
        if sig in self._lru:
            plan.admission = ADMISSION_REPLAY
        else:
            plan.miss_reason = self._planner.attribute_miss_reason(layers, list(self._lru.values()))
        return plan

    def admit_for_call(self, plan: GraphPlan):
        """Account for the call and return the cache's capture scope for its signature."""
        sig = plan.signature
        if sig in self._lru:
            self._lru.move_to_end(sig)
            self._hits += 1
            plan.admission = ADMISSION_REPLAY
        else:
            self._misses += 1
            reason = plan.miss_reason or "no_entry"
            self._miss_reasons[reason] = self._miss_reasons.get(reason, 0) + 1
            if self._cache.is_frozen():
                raise RuntimeError(f"graph cache is READY (frozen): new signature refused ({reason}); "
                                   f"{self._cache.explain_miss(sig)}")
            while len(self._lru) >= self._max:
                old, _ = self._lru.popitem(last=False)
                self._cache.evict(old)
                self._evict_total += 1
                plan.evicted.append(getattr(old, "_impl", None))
                plan.lifecycle = LIFECYCLE_EVICT
            self._lru[sig] = plan.layers
            plan.admission = ADMISSION_RECORD
        return self._cache.capture(sig)

    def touch_after_call(self, plan: GraphPlan, in_scope_state: int) -> None:
        """A scope that ended in pass-through is forgotten so the next call records again."""
        from ._runtime import STATE_PASSTHROUGH
        if in_scope_state == STATE_PASSTHROUGH and plan.signature in self._lru:
            del self._lru[plan.signature]
            plan.admission = ADMISSION_RECAPTURE

    def stats(self) -> Dict[str, Any]:
        return {"entries": len(self._lru), "max_entries": self._max, "hits": self._hits, "misses": self._misses,
                "evictions": self._evict_total, "miss_reasons": dict(self._miss_reasons),
                "backend_entries": self._cache.size()}

    def clear(self) -> None:
        self._lru.clear()
        self._cache.clear()


__all__ = ["SignaturePlanner", "SignatureLayers", "GraphPlan", "EntryRegistry", "MISS_REASONS", "WORKLOAD_KINDS",
           "ADMISSION_KINDS", "WORKLOAD_PREFILL", "WORKLOAD_DECODE", "WORKLOAD_GENERIC"]
