"""Diagnostics behind ``torch.rpu``: wrapper counters, debug-tensor export, kernel-trace scopes.

Three mechanisms mirror the reference (``docs/runtime_config.md:464-474``): (1) launch counters
(``set_profile`` / ``profile_counters`` -- here the native library's launch counter), (2)
``torch.profiler`` ranges named after graph signatures (emitted by the capture scopes), (3) a
per-scope kernel trace: the reference dumps hardware cycle traces per graph segment
(``python/rpu_backend/runtime/debug.py:76-133``); here ``hw_perf_trace(dir)`` wraps the scope in a
CUDA-activity ``torch.profiler`` session and writes one Chrome trace per scope, budgeted by
``max_dumps``.
"""
from __future__ import annotations

import contextlib
import os
import threading
from typing import Dict, Optional

_debug = False
_profile = False
_export = False
_spm_debug = False
_tensors: Dict[str, object] = {}
_profile_base = 0
_hw = {"dir": None, "max_dumps": 0, "seq": 0}
_lock = threading.Lock()


def set_debug(enabled: bool) -> None:
    global _debug
    _debug = bool(enabled)


def get_debug() -> bool:
    return _debug


def _launches() -> int:
    from .. import _native
    if not _native.available():
        return 0
    import ctypes
    lib = _native.lib()
    lib.rf_launch_count.restype = ctypes.c_uint64
    return int(lib.rf_launch_count())


def set_profile(enabled: bool) -> None:
    global _profile, _profile_base
    _profile = bool(enabled)
    if _profile:
        _profile_base = _launches()


def get_profile() -> bool:
    return _profile


def reset_profile_accumulators() -> None:
    global _profile_base
    _profile_base = _launches()


def profile_counters() -> dict:
    return {"kernel_launches": _launches() - _profile_base if _profile else 0}


def set_debug_export(enabled: bool) -> None:
    global _export
    _export = bool(enabled)
    if not _export:
        _tensors.clear()


def get_debug_export() -> bool:
    return _export


def export_debug_tensor(name: str, tensor) -> None:
    """Called by runtimes at probe points; keeps a detached host copy when export is on."""
    if _export:
        _tensors[name] = tensor.detach().to("cpu").clone()


def get_debug_tensor(name: str):
    return _tensors.get(name)


def list_debug_tensors() -> list:
    """Names of the probe tensors held since export was switched on, in export order."""
    return list(_tensors)


def clear_debug_tensors() -> None:
    _tensors.clear()


def set_spm_debug(enabled: bool) -> None:
    global _spm_debug
    _spm_debug = bool(enabled)


def get_spm_debug() -> bool:
    return _spm_debug


def spm_alloc_dump() -> str:
    """Arena / pool occupancy in place of the reference's scratch-pad dump."""
    from .control import memory_stats
    s = memory_stats()
    return (f"device memory: allocated={s['allocated_bytes']} reserved={s['reserved_bytes']} "
            f"peak={s['peak_allocated_bytes']}")


def set_hw_perf_trace(output_dir: Optional[str], max_dumps: int = 8) -> None:
    with _lock:
        _hw["dir"], _hw["max_dumps"], _hw["seq"] = (str(output_dir) if output_dir else None), int(max_dumps), 0
        if output_dir:
            os.makedirs(output_dir, exist_ok=True)


def get_hw_perf_trace() -> dict:
    """``{"dir", "max_dumps", "seq"}`` of the trace configuration in force (``dir`` is None when tracing is off)."""
    with _lock:
        return {"dir": _hw.get("dir"), "max_dumps": _hw.get("max_dumps", 0), "seq": _hw.get("seq", 0)}


@contextlib.contextmanager
def hw_perf_trace(output_dir: str, max_dumps: int = 8, name: str = "scope"):
    """Trace the kernels launched inside the ``with`` block into
    ``rpu_hwperf_pid<P>_tid<T>_seq<S>_<name>.json`` (Chrome trace), at most ``max_dumps`` files."""
    import torch
    set_hw_perf_trace(output_dir, max_dumps)
    prof = None
    try:
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        prof = torch.profiler.profile(activities=acts)
        prof.__enter__()
        yield
    finally:
        try:
            if prof is not None:
                prof.__exit__(None, None, None)
                with _lock:
                    if _hw["seq"] < _hw["max_dumps"]:
                        path = os.path.join(output_dir, f"rpu_hwperf_pid{os.getpid()}_tid{threading.get_ident()}_"
                                                        f"seq{_hw['seq']}_{name}.json")
                        prof.export_chrome_trace(path)
                        _hw["seq"] += 1
        finally:
            set_hw_perf_trace(None, 0)
