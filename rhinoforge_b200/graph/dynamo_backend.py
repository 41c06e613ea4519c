"""A TorchDynamo backend over the CUDA-graph runtime: Dynamo traces, this package captures and replays.

    compiled = torch.compile(module, backend=dynamo_backend)            # process-wide backend object
    be = RpuDynamoBackend(max_entries=2); m1 = torch.compile(m1, backend=be); m2 = torch.compile(m2, backend=be)

``torch.compile`` is a *front-end* here, never the code generator: the traced FX graph runs exactly the eager kernels.
Per traced graph module the backend

1. checks that no opted-in sub-module still creates state at its first forward (``lazy_init_guard``);
2. cuts the graph into runs that can be stream-captured and nodes that talk to the host
   (:func:`rhinoforge_b200.graph.dynamo_partitioner.partition_for_capture`);
3. on each call builds the call's signature; a new signature records one :class:`GraphCapture` per capturable run (a CUDA
   graph with static input buffers), a known one replays them.  Signatures live in an LRU of ``max_entries`` per
   backend: the coldest entry is invalidated - its graph and buffers freed - before a new one is recorded.

The bound matters.  A decode loop whose position is a Python integer makes Dynamo re-trace every step (the integer is
guarded), so every step arrives as a new graph module; with an unbounded table each of them would pin a captured graph
and its buffers.  ``max_entries=1`` keeps one; raise it to 2-4 when prefill and decode signatures alternate.

Model runtimes of this package capture their own graphs and must not be wrapped in ``torch.compile`` as well (nested
capture is refused by CUDA); the backend is for user code around them and for experiments, as in the reference, where it
is likewise not a production path (``python/rpu_backend/graph/dynamo_backend.py:1-60``).  Without a CUDA device every
capture is pass-through and the backend degrades to running the traced graph eagerly.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ._runtime import GraphCache
from .admission import SignaturePlanner
from .dynamo_partitioner import Partitioned, partition_for_capture
from .lazy_init_guard import verify_graph_module_best_effort
from .manual_capture import GraphCapture


class _Entry:
    """Everything recorded for one (graph module, signature): a capture per capturable segment."""

    def __init__(self) -> None:
        self.captures: Dict[str, GraphCapture] = {}

    def invalidate(self) -> None:
        for c in self.captures.values():
            c.invalidate()
        self.captures.clear()


class RpuDynamoBackend:
    def __init__(self, *, max_entries: int = 1, cache: Optional[GraphCache] = None, partition: bool = True,
                 is_capturable: Optional[Callable[[torch.fx.Node], bool]] = None):
        if max_entries < 1:
            raise ValueError("max_entries must be positive (an unbounded table pins one captured graph per re-trace)")
        self.max_entries = int(max_entries)
        self._cache = cache
        self._partition = partition
        self._is_capturable = is_capturable
        self._planner = SignaturePlanner()
        self._lru: "OrderedDict[Tuple[int, Any], _Entry]" = OrderedDict()
        self._counters = {"graphs": 0, "records": 0, "replays": 0, "evictions": 0, "segments": 0, "host_segments": 0}

    # ------------------------------------------------------------------ Dynamo entry point
    def __call__(self, gm: torch.fx.GraphModule, example_inputs: Sequence[Any]) -> Callable[..., Any]:
        verify_graph_module_best_effort(gm, example_inputs)
        self._counters["graphs"] += 1
        gm_key = self._counters["graphs"]
        parts: Optional[Partitioned] = None
        if self._partition:
            parts = partition_for_capture(gm, self._is_capturable)
            self._counters["segments"] += len(parts.segments)
            self._counters["host_segments"] += sum(1 for s in parts.segments if not s.capturable)
            if all(s.capturable for s in parts.segments) and len(parts.segments) <= 1:
                parts = None                                   # one capturable run: capture the module as a whole
        backend = self

        def compiled_call(*args: Any) -> Any:
            layers = backend._planner.layers_for_call(f"dynamo:{gm_key}", args, {})
            key = (gm_key, layers)
            entry = backend._lru.get(key)
            if entry is None:
                while len(backend._lru) >= backend.max_entries:
                    _, old = backend._lru.popitem(last=False)
                    old.invalidate()
                    backend._counters["evictions"] += 1
                entry = backend._lru[key] = _Entry()
                backend._counters["records"] += 1
            else:
                backend._lru.move_to_end(key)
                backend._counters["replays"] += 1
            if parts is None:
                return backend._run_segment(entry, "<whole>", gm_key, 0, gm.forward, args)
            return parts.run(args, lambda i, seg, fn, seg_args: (
                backend._run_segment(entry, seg.name, gm_key, i + 1, fn, seg_args) if seg.capturable else fn(*seg_args)))

        compiled_call.__wrapped__ = gm.forward                 # type: ignore[attr-defined]
        return compiled_call

    def _run_segment(self, entry: _Entry, name: str, gm_key: int, segment: int, fn: Callable[..., Any],
                     args: Sequence[Any]) -> Any:
        cap = entry.captures.get(name)
        if cap is None:
            cap = entry.captures[name] = GraphCapture(fn, tuple(args), cache=self._cache,
                                                      op_id=f"dynamo:{gm_key}:{name}", segment=segment)
            return cap.cached_output
        return cap.replay(*args)

    # ------------------------------------------------------------------ management
    def stats(self) -> Dict[str, Any]:
        return {**self._counters, "entries": len(self._lru), "max_entries": self.max_entries}

    def clear(self) -> None:
        """Invalidate every recorded entry (captured graphs and their static buffers are released)."""
        for e in self._lru.values():
            e.invalidate()
        self._lru.clear()

    def __repr__(self) -> str:
        return f"RpuDynamoBackend(max_entries={self.max_entries}, entries={len(self._lru)})"


dynamo_backend = RpuDynamoBackend()

__all__ = ["RpuDynamoBackend", "dynamo_backend"]
