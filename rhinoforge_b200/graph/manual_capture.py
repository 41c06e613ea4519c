"""Manual capture: ``g = capture(fn, x, y); out = g.replay(x2, y2)`` in the style of a CUDA graph.

One :class:`GraphCapture` owns one entry of a :class:`GraphCache`.  Construction runs ``fn`` once inside the
cache's capture scope (stream capture of every kernel it launches, then one launch), keeps the example inputs as the
graph's *static input buffers* and the returned tensors as its *static outputs*.  ``replay(*args)`` checks that the new
arguments have the signature that was captured - a changed shape, dtype, layout or scalar is refused with the name of
the first differing layer, never silently re-captured - copies tensor arguments into the static buffers (skipped for
an argument that already is the buffer) and launches the graph.  Reference behaviour:
``python/rpu_backend/graph/manual_capture.py:33-160,287-346`` (eager recording at construction, drift refusal,
``dynamic_inputs`` not supported).

Without a CUDA device or the native library the object degrades to *pass-through*: ``replay`` simply calls ``fn``;
``replayable`` is False and ``non_replayable_reason`` says why.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from ._runtime import STATE_BUILT, GraphCache, GraphSignature, backend_loaded
from .admission import SignaturePlanner


def _tensors_of(obj: Any, out: List[torch.Tensor]) -> None:
    if isinstance(obj, torch.Tensor):
        out.append(obj)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            _tensors_of(v, out)
    elif isinstance(obj, dict):
        for k in sorted(obj, key=str):
            _tensors_of(obj[k], out)


class GraphCapture:
    def __init__(self, fn: Callable[..., Any], example_args: Sequence[Any] = (),
                 example_kwargs: Optional[Dict[str, Any]] = None, *, cache: Optional[GraphCache] = None,
                 op_id: Optional[str] = None, segment: int = 0, dynamic_inputs: Sequence[str] = ()):
        if dynamic_inputs:
            raise NotImplementedError("dynamic_inputs (patching captured arguments at replay) is not supported: "
                                      "inputs are static buffers that replay() refills")
        self._fn = fn
        self._args, self._kwargs = tuple(example_args), dict(example_kwargs or {})
        self._planner = SignaturePlanner()
        self._op_id = op_id or f"manual:{getattr(fn, '__module__', '')}.{getattr(fn, '__qualname__', type(fn).__qualname__)}"
        self._segment = segment
        self._sig, self._layers = self._planner.build_signature(self._op_id, self._args, self._kwargs, branch=fn,
                                                                segment=segment)
        self._static_inputs: List[torch.Tensor] = []
        _tensors_of((self._args, self._kwargs), self._static_inputs)
        self._cache = cache
        self._reason = ""
        self._replays = 0
        self._passthrough_calls = 0
        self._valid = True
        on_gpu = backend_loaded() and torch.cuda.is_available() and all(t.is_cuda for t in self._static_inputs)
        if not on_gpu:
            self._reason = ("native graph backend not loaded" if not backend_loaded() else
                            "no CUDA device" if not torch.cuda.is_available() else "an input tensor is not on the GPU")
            self._output = fn(*self._args, **self._kwargs)
            return
        if self._cache is None:
            self._cache = GraphCache()
        if self._cache.lookup(self._sig) is not None:
            raise RuntimeError(f"the cache already holds an entry for {self._sig!r}: one GraphCapture per signature")
        with self._cache.capture(self._sig) as handle:
            if handle is None or not handle.recording:
                raise RuntimeError("manual capture expected a recording scope")
            self._output = fn(*self._args, **self._kwargs)
        entry = self._snapshot_entry()
        if not entry or entry.get("state") != STATE_BUILT or entry.get("non_replayable"):
            self._reason = (entry or {}).get("non_replayable_reason") or "capture did not reach the BUILT state"

    # ------------------------------------------------------------------ replay
    def replay(self, *args: Any, **kwargs: Any) -> Any:
        if not self._valid:
            raise RuntimeError("this GraphCapture was invalidated")
        if not args and not kwargs:
            args, kwargs = self._args, self._kwargs
        elif args is not self._args or kwargs:
            _, layers = self._planner.build_signature(self._op_id, args, kwargs, branch=self._fn, segment=self._segment)
            where = layers.first_divergence(self._layers)
            if where is not None:
                raise RuntimeError(f"replay arguments differ from the captured call in {where}; capture a new graph "
                                   "for this signature (no silent recapture)")
        if not self.replayable:
            self._passthrough_calls += 1
            return self._fn(*args, **kwargs)
        fresh: List[torch.Tensor] = []
        _tensors_of((tuple(args), dict(kwargs)), fresh)
        for dst, src in zip(self._static_inputs, fresh):
            if dst is not src and dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self._cache.replay(self._sig)
        self._replays += 1
        return self._output

    __call__ = replay

    def invalidate(self) -> None:
        """Drop the cache entry; the object cannot replay afterwards."""
        if self._valid and self._cache is not None and not self._reason:
            self._cache.evict(self._sig)
        self._valid = False

    # ------------------------------------------------------------------ introspection
    @property
    def signature(self) -> GraphSignature:
        return self._sig

    @property
    def cache(self) -> Optional[GraphCache]:
        return self._cache

    @property
    def cached_output(self) -> Any:
        return self._output

    @property
    def replayable(self) -> bool:
        return self._valid and not self._reason

    @property
    def non_replayable_reason(self) -> str:
        return self._reason if self._valid else "invalidated"

    def _snapshot_entry(self) -> Optional[dict]:
        if self._cache is None or self._sig._impl is None:
            return None
        for e in self._cache.snapshot():
            if e["signature"] == self._sig._impl:
                return e
        return None

    def stats(self) -> Dict[str, Any]:
        e = self._snapshot_entry() or {}
        return {"replayable": self.replayable, "non_replayable_reason": self.non_replayable_reason,
                "replays": self._replays, "passthrough_calls": self._passthrough_calls,
                "static_inputs": len(self._static_inputs), "node_count": e.get("node_count", 0),
                "kernel_count": e.get("kernel_count", 0), "build_count": e.get("build_count", 0),
                "backend_replay_count": e.get("replay_count", 0)}

    def __repr__(self) -> str:
        return (f"GraphCapture({self._op_id!r}, replayable={self.replayable}, replays={self._replays}"
                + (f", reason={self._reason!r}" if self._reason else "") + ")")


def capture(fn: Callable[..., Any], *example_args: Any, cache: Optional[GraphCache] = None, op_id: Optional[str] = None,
            segment: int = 0, dynamic_inputs: Sequence[str] = (), **example_kwargs: Any) -> GraphCapture:
    """Capture ``fn(*example_args, **example_kwargs)``; see :class:`GraphCapture`."""
    return GraphCapture(fn, example_args, example_kwargs, cache=cache, op_id=op_id, segment=segment,
                        dynamic_inputs=dynamic_inputs)


__all__ = ["GraphCapture", "capture"]
