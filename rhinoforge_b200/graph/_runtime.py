"""``GraphSignature`` / ``GraphCache``: the Python face of the native CUDA-graph cache.

A cache moves through CONFIGURING -> WARMING -> READY.  ``with cache.capture(sig):`` runs its
body once in BUILD mode (stream capture; the graph is launched at scope exit) and afterwards in
REPLAY mode (the body's native launches are skipped, the stored graph is launched at scope
exit).  READY forbids new BUILDs and evictions.  Without a CUDA device the wrappers stay inert:
signatures compare equal only by identity of "no backend", scopes do nothing, ``freeze`` raises.

Semantics follow ``python/rpu_backend/graph/_runtime.py:49-340``; the native half is
``csrc/runtime/graph_exec.cpp``.
"""
from __future__ import annotations

import ctypes as C
import threading
import warnings
import weakref
from typing import Any, List, Optional

import torch

_backend = None          # the loaded native library, or None (host-only)
_LIVE: "weakref.WeakSet[GraphCache]" = weakref.WeakSet()
_tls = threading.local()

STATE_PASSTHROUGH, STATE_RECORDING, STATE_BUILT, STATE_REPLAYING = 0, 1, 2, 3

_DTYPE_CODE = {torch.float16: 5, torch.bfloat16: 15, torch.float32: 6, torch.int32: 3, torch.int64: 4, torch.bool: 11,
               torch.int8: 1, torch.uint8: 0}


def configure_backend(lib: Any = None, tag: Optional[str] = None) -> None:
    """Bind (or unbind) the native library before any real graph object exists."""
    global _backend
    _backend = lib


def backend_loaded() -> bool:
    return _backend is not None


def fnv1a_64(text: str) -> int:
    """Signed 64-bit FNV-1a of ``text`` -- the numeric operation id of a signature."""
    h = 0xCBF29CE484222325
    for b in text.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h - (1 << 64) if h >= (1 << 63) else h


class GraphSignature:
    """Structured key of one cache entry: operation id, shapes, dynamic dims, dtypes, flags,
    branch key, segment key."""

    def __init__(self, op_id="", shapes=(), dyn_dims=(), dtypes=(), flags=0, branch_key=0, segment_key=0):
        self.op_id = str(op_id) if isinstance(op_id, (str, int)) else ""
        if not backend_loaded():
            self._impl = None
            return
        oid = fnv1a_64(op_id) if isinstance(op_id, str) else int(op_id)
        dts = [(_DTYPE_CODE[d] if isinstance(d, torch.dtype) else int(d)) for d in dtypes]
        sh, dy = [int(v) for v in shapes], [int(v) for v in dyn_dims]
        self._impl = tuple([oid, int(flags), int(branch_key), int(segment_key), len(sh), *sh, len(dy), *dy,
                            len(dts), *dts])

    def _words(self):
        arr = (C.c_int64 * len(self._impl))(*self._impl)
        return arr, len(self._impl)

    def __repr__(self) -> str:
        return f"GraphSignature({self.op_id!r}, {self._impl})" if self._impl is not None else \
            "GraphSignature(<no backend>)"

    def __eq__(self, other):
        if not isinstance(other, GraphSignature):
            return NotImplemented
        return self._impl == other._impl

    def __hash__(self):
        return hash(self._impl) if self._impl is not None else 0


class GraphHandle:
    """What a capture scope yields: the state it runs in and the entry's counters."""

    def __init__(self, cache: "GraphCache", sig: GraphSignature, state: int):
        self._cache, self._sig, self._state = cache, sig, state

    def state(self) -> int:
        return self._state

    @property
    def recording(self) -> bool:
        return self._state == STATE_RECORDING

    @property
    def replaying(self) -> bool:
        return self._state == STATE_REPLAYING

    def debug_stats(self) -> dict:
        for e in self._cache.snapshot():
            if e["signature"] == self._sig._impl:
                return e
        return {}


def _skip_idle_record_function() -> bool:
    from ..runtime.control import rpu_env_bool
    if not rpu_env_bool("RPU_SKIP_IDLE_RECORD_FUNCTION", False):
        return False
    try:
        return not torch.autograd._profiler_enabled()
    except Exception:  # noqa: BLE001
        return False


class _CaptureScope:
    def __init__(self, cache: "GraphCache", sig: GraphSignature, stream=None):
        self._cache, self._sig, self._stream = cache, sig, stream
        self._open = False
        self._prof = None
        self._torch_stream_ctx = None

    def __enter__(self):
        c = self._cache
        if c._impl is None or self._sig._impl is None:
            return None
        allow = 0 if c.is_frozen() else 1
        if self._stream is None:
            # capture needs a non-default stream
            cur = torch.cuda.current_stream()
            if cur == torch.cuda.default_stream():
                c._side_stream.wait_stream(cur)
                self._torch_stream_ctx = torch.cuda.stream(c._side_stream)
                self._torch_stream_ctx.__enter__()
            self._stream = torch.cuda.current_stream()
        words, n = self._sig._words()
        st = C.c_int32(0)
        rc = _backend.rf_graph_begin(c._impl, words, n, C.c_void_p(self._stream.cuda_stream), allow, C.byref(st))
        if rc != 0:
            self._leave_stream()
            msg = _backend.rf_last_error().decode(errors="replace")
            raise RuntimeError(f"GraphCache {'READY miss' if not allow else 'begin failed'} for {self._sig!r}: {msg}")
        self._open = True
        if not _skip_idle_record_function():
            try:
                from torch.profiler import record_function
                self._prof = record_function(self._sig.op_id or "rpu_graph_capture")
                self._prof.__enter__()
            except Exception:  # noqa: BLE001
                self._prof = None
        return GraphHandle(c, self._sig, st.value)

    def _leave_stream(self):
        if self._torch_stream_ctx is not None:
            side = torch.cuda.current_stream()
            self._torch_stream_ctx.__exit__(None, None, None)
            torch.cuda.current_stream().wait_stream(side)
            self._torch_stream_ctx = None

    def __exit__(self, et, ev, tb):
        try:
            if not self._open:
                return False
            if et is None:
                rc = _backend.rf_graph_end(self._cache._impl)
                if rc != 0:
                    msg = _backend.rf_last_error().decode(errors="replace")
                    _backend.rf_graph_abort(self._cache._impl)
                    raise RuntimeError(f"graph end failed for {self._sig!r}: {msg}")
            else:
                _backend.rf_graph_abort(self._cache._impl)
            return False
        finally:
            self._leave_stream()
            if self._prof is not None:
                self._prof.__exit__(et, ev, tb)
                self._prof = None


class GraphCache:
    """Signature-indexed cache of captured graphs with CONFIGURING / WARMING / READY phases."""

    DEFAULT_MAX_ENTRIES = 32
    _CONFIGURING, _WARMING, _READY = "CONFIGURING", "WARMING", "READY"

    def __init__(self, max_entries: Optional[int] = None):
        self._phase = self._CONFIGURING
        self._impl = None
        if not backend_loaded():
            return
        n = self.DEFAULT_MAX_ENTRIES if max_entries is None else int(max_entries)
        self._impl = C.c_int64(_backend.rf_graphcache_create(n))
        self._side_stream = torch.cuda.Stream()
        _LIVE.add(self)

    def __del__(self):
        try:
            if self._impl is not None and _backend is not None:
                _backend.rf_graphcache_destroy(self._impl)
        except Exception:  # noqa: BLE001
            pass

    def capture(self, sig: GraphSignature, stream=None):
        return _CaptureScope(self, sig, stream)

    def replay(self, sig: GraphSignature, stream=None) -> None:
        """Launch a built entry directly (no host re-walk)."""
        if self._impl is None:
            raise RuntimeError("GraphCache.replay requires the C++ backend")
        words, n = sig._words()
        s = stream or torch.cuda.current_stream()
        if _backend.rf_graph_replay(self._impl, words, n, C.c_void_p(s.cuda_stream)) != 0:
            raise RuntimeError(_backend.rf_last_error().decode(errors="replace"))

    def begin_warmup(self):
        self._phase = self._WARMING
        return self

    def freeze(self):
        if self._impl is None:
            raise RuntimeError("GraphCache.freeze requires the C++ backend")
        entries = self.snapshot()
        if not entries:
            raise RuntimeError("GraphCache.freeze requires at least one prewarmed BUILT entry")
        for e in entries:
            if e["state"] != STATE_BUILT:
                raise RuntimeError(f"GraphCache READY entry is not BUILT (state={e['state']}); "
                                   "online recapture is disabled")
            if e["non_replayable"]:
                raise RuntimeError("GraphCache READY entry is non-replayable")
        self._phase = self._READY
        return self

    def is_frozen(self) -> bool:
        return self._phase == self._READY

    @property
    def phase(self) -> str:
        return self._phase

    def lookup(self, sig: GraphSignature):
        if self._impl is None:
            return None
        words, n = sig._words()
        st = _backend.rf_graphcache_lookup(self._impl, words, n)
        return None if st < 0 else GraphHandle(self, sig, st)

    def get_or_create(self, sig):
        return self.lookup(sig)

    def evict(self, sig: GraphSignature) -> None:
        if self.is_frozen():
            raise RuntimeError("GraphCache READY entries cannot be evicted; call begin_warmup() first")
        if self._impl is not None:
            words, n = sig._words()
            _backend.rf_graphcache_evict(self._impl, words, n)

    def clear(self) -> None:
        if self._impl is not None:
            _backend.rf_graphcache_clear(self._impl)

    def size(self) -> int:
        return _backend.rf_graphcache_size(self._impl) if self._impl is not None else 0

    def max_entries(self) -> int:
        return _backend.rf_graphcache_max_entries(self._impl) if self._impl is not None else 0

    def snapshot(self) -> List[dict]:
        if self._impl is None:
            return []
        buf = C.create_string_buffer(1 << 16)
        _backend.rf_graphcache_snapshot(self._impl, buf, len(buf))
        out = []
        for line in buf.value.decode().splitlines():
            head, words = line.split("|", 1)
            f = head.split()
            out.append({"op_id": int(f[0]), "state": int(f[1]), "build_count": int(f[2]), "replay_count": int(f[3]),
                        "recapture_count": int(f[4]), "node_count": int(f[5]), "kernel_count": int(f[6]),
                        "non_replayable": f[7] != "-", "non_replayable_reason": "" if f[7] == "-" else f[7],
                        "signature": tuple(int(w) for w in words.split(",") if w)})
        return out

    def cache_invariant_ok(self) -> bool:
        return bool(_backend.rf_graphcache_invariant_ok(self._impl)) if self._impl is not None else True

    def touch_entry(self, sig, replay: bool) -> None:  # counters are kept natively
        return None

    def debug_bucket_counts(self) -> dict:
        out: dict = {}
        for e in self.snapshot():
            key = e["signature"][4:]
            out[key] = out.get(key, 0) + 1
        return out

    def debug_branch_counts(self) -> dict:
        out: dict = {}
        for e in self.snapshot():
            out[e["signature"][2]] = out.get(e["signature"][2], 0) + 1
        return out

    def dump_signature_tree(self) -> str:
        snap = self.snapshot()
        if not snap:
            return "<empty>"
        return "\n".join(f"op {e['op_id']} state {e['state']} builds {e['build_count']} replays {e['replay_count']} "
                         f"sig {e['signature']}" for e in snap)

    def explain_miss(self, sig: GraphSignature) -> str:
        if self._impl is None:
            return "miss at GmId: backend unavailable"
        words, n = sig._words()
        buf = C.create_string_buffer(1024)
        _backend.rf_graphcache_explain_miss(self._impl, words, n, buf, len(buf))
        return buf.value.decode()

    @classmethod
    def clear_all(cls) -> None:
        for cache in list(_LIVE):
            try:
                cache.clear()
            except Exception as exc:  # noqa: BLE001
                warnings.warn(f"GraphCache.clear_all: clear failed for one instance: {type(exc).__name__}: {exc}",
                              stacklevel=2)


def get_default_graph_cache() -> GraphCache:
    cached = getattr(_tls, "cache", None)
    if cached is None:
        cached = _tls.cache = GraphCache()
    return cached


def reset_graph_cache() -> None:
    """Drop every entry of every live cache (public top-level helper)."""
    GraphCache.clear_all()


def install_torch_namespace(mod: Any) -> None:
    mod.GraphCache = GraphCache
    mod.GraphSignature = GraphSignature
    mod.get_default_graph_cache = get_default_graph_cache


__all__ = ["GraphCache", "GraphSignature", "GraphHandle", "configure_backend", "get_default_graph_cache",
           "install_torch_namespace", "reset_graph_cache", "backend_loaded"]
