"""The ``torch.rpu`` namespace: a torch.cuda-shaped device protocol plus runtime controls.

``rpu`` names the B200 the process runs on; everything here is a thin shim over the CUDA runtime
(reference surface: ``python/rpu_backend/_torch_rpu.py:7-75``, ``docs/api_reference.md:301-337``).
"""
from __future__ import annotations

import sys
import types


def _backend_ready() -> bool:
    import torch
    from . import _native
    return bool(torch.cuda.is_available()) and _native.available()


def configure_torch_rpu(torch, mod: types.ModuleType):
    from .runtime import control, debug, log
    mod.is_available = _backend_ready
    mod.device_count = lambda: (torch.cuda.device_count() if torch.cuda.is_available() else 0)
    mod.current_device = lambda: (torch.cuda.current_device() if torch.cuda.is_available() else 0)
    mod.set_device = lambda i: torch.cuda.set_device(i)
    mod.synchronize = lambda device=None: torch.cuda.synchronize(device) if torch.cuda.is_available() else None
    mod.manual_seed_all = lambda seed: torch.cuda.manual_seed_all(seed) if torch.cuda.is_available() else None
    mod.manual_seed = mod.manual_seed_all
    mod.is_initialized = lambda: torch.cuda.is_initialized()
    mod._is_in_bad_fork = lambda: torch.cuda._is_in_bad_fork() if hasattr(torch.cuda, "_is_in_bad_fork") else False
    mod.get_device_name = lambda i=None: torch.cuda.get_device_name(i) if torch.cuda.is_available() else "cpu"
    for name in ("set_caching_allocator", "get_caching_allocator", "empty_cache", "memory_stats",
                 "reset_peak_memory_stats", "set_ddr_flush", "set_ddr_flush_force", "set_cross_layer_batch_size",
                 "set_cross_layer_batch_prefill", "get_cross_layer_batch_size", "shutdown", "get_ddr_flush",
                 "get_ddr_flush_force", "get_amp_supported_dtype", "is_autocast_available", "get_spm_mode",
                 "get_allreduce_twostage", "get_linear_acc32", "get_memory_stats", "reset_accumulated_memory_stats",
                 "get_cross_layer_batch_prefill", "spm_alloc_reset_temporary", "reset_temporary_spm", "reset_all_spm"):
        setattr(mod, name, getattr(control, name))
    for name in ("set_debug_level", "get_debug_level"):
        setattr(mod, name, getattr(log, name))
    for name in ("set_debug", "get_debug", "set_profile", "get_profile", "reset_profile_accumulators",
                 "set_debug_export", "get_debug_export", "get_debug_tensor", "set_spm_debug", "spm_alloc_dump",
                 "set_hw_perf_trace", "hw_perf_trace", "profile_counters", "get_hw_perf_trace", "list_debug_tensors",
                 "clear_debug_tensors", "get_spm_debug"):
        setattr(mod, name, getattr(debug, name))
    return control


def install(torch) -> types.ModuleType:
    if "torch.rpu" in sys.modules:
        mod = sys.modules["torch.rpu"]
    else:
        mod = types.ModuleType("torch.rpu")
        mod.__dict__["__file__"] = "<rhinoforge_b200 dynamic>"
        sys.modules["torch.rpu"] = mod
        torch.rpu = mod
    return mod
