"""Runtime controls behind ``torch.rpu``: the one strict boolean environment parser, allocator and
memory statistics (thin shims over the CUDA caching allocator), warm-up count, shutdown.

The reference's tile / scratch-pad / DMA selectors have no meaning on B200 and are not read; the
variables that keep their meaning are listed in ``KEPT_ENV`` and parsed only here
(reference: ``python/rpu_backend/runtime/control.py:47-61,281-323``, ``docs/runtime_config.md:14-40``).
"""
from __future__ import annotations

import os
from typing import Dict

_TRUE = frozenset({"1", "true", "on"})
_FALSE = frozenset({"0", "false", "off", ""})

# name -> (kind, default, lifecycle)
KEPT_ENV: Dict[str, tuple] = {
    "RPU_MODEL_CACHE": ("path", None, "IMPORT"),
    "RPU_LOG_LEVEL": ("int", 3, "IMPORT"),
    "RPU_WARMUP": ("int", 0, "CALL"),
    "RPU_CAUSAL_PREFILL_PADDING_BUDGET": ("int", 64, "MODEL"),
    "RPU_SKIP_IDLE_RECORD_FUNCTION": ("bool", False, "CALL"),
    "RPU_TP_COMM": ("enum:fused,nccl", "fused", "MODEL"),
    "RPU_PI05_FUSED_DENOISE": ("bool", True, "MODEL"),
    "RPU_PI05_DENOISE_UNROLL": ("bool", True, "MODEL"),
    "RPU_LINGBOT2_DENOISE_UNROLL": ("bool", True, "MODEL"),
    "RPU_WALL_OSS_FUSED_DENOISE": ("bool", True, "MODEL"),
    "RPU_HY_VLA_UNROLL": ("bool", True, "MODEL"),
    "RPU_QWEN3_5_FREE_HF_WEIGHTS": ("bool", False, "MODEL"),
    "QWEN3_5_TEXT_CHUNK": ("int", 0, "MODEL"),
    "QWEN3_5_TEXT_PADDING_BUDGET": ("int", 64, "MODEL"),
    "QWEN3_VL_32B_ALLOW_GRAPH_BLOCKED": ("exact1", False, "MODEL"),
    "RF_B200_NO_BUILD": ("exact1", False, "IMPORT"),
}

# variables of the reference that are dropped here and refused in run configs
DROPPED_ENV = frozenset({"RPU_KERNEL_LIB_PATH", "LKN_MAX_BATCH_ENTRIES", "LKN_KD_BUF_MB", "LKN_INSTR_BUF_MB"})


def rpu_env_bool(name: str, default: bool = False, *, cpp_mirror=None) -> bool:
    """The only boolean environment reader.  unset -> default; 1/true/on -> True;
    0/false/off/'' -> False (case-insensitive, stripped); anything else raises ``ValueError``
    so that a typo cannot silently select the wrong path."""
    raw = os.environ.get(name)
    if raw is None:
        return default
    v = raw.strip().lower()
    if cpp_mirror is not None and raw.strip() not in ("0", "1"):
        raise ValueError(f"{name} is also read by native code ({cpp_mirror}); set it to 1 or 0, got {raw!r}.")
    if v in _TRUE:
        return True
    if v in _FALSE:
        return False
    raise ValueError(f"{name} must be one of 1/0, true/false, or on/off (case-insensitive); got {raw!r}.")


def rpu_env_exact1(name: str) -> bool:
    """Fail-closed opt-in gates: only the exact literal ``1`` enables."""
    return os.environ.get(name) == "1"


def rpu_env_int(name: str, default: int, *, minimum: int = 0) -> int:
    raw = os.environ.get(name)
    if raw is None or raw.strip() == "":
        return default
    try:
        v = int(raw.strip())
    except ValueError as e:
        raise ValueError(f"{name} must be an integer, got {raw!r}") from e
    if v < minimum:
        raise ValueError(f"{name} must be >= {minimum}, got {v}")
    return v


def warmup_iters() -> int:
    return rpu_env_int("RPU_WARMUP", 0)


def tp_comm_mode() -> str:
    v = os.environ.get("RPU_TP_COMM", "fused").strip().lower()
    if v not in ("fused", "nccl"):
        raise ValueError(f"RPU_TP_COMM must be 'fused' or 'nccl', got {v!r}")
    return v


# ---- allocator / memory (CUDA caching allocator underneath) -----------------------------------
_caching = True
_flush = False
_cross_layer_batch = 0


def set_caching_allocator(enabled: bool) -> None:
    """Kept for API compatibility; device memory always comes from PyTorch's CUDA caching allocator
    plus the static arenas, so this only records the request."""
    global _caching
    _caching = bool(enabled)


def get_caching_allocator() -> bool:
    return _caching


def empty_cache() -> None:
    import torch
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def memory_stats() -> dict:
    import torch
    if not torch.cuda.is_available():
        return {"allocated_bytes": 0, "reserved_bytes": 0, "peak_allocated_bytes": 0}
    return {"allocated_bytes": torch.cuda.memory_allocated(), "reserved_bytes": torch.cuda.memory_reserved(),
            "peak_allocated_bytes": torch.cuda.max_memory_allocated()}


def reset_peak_memory_stats() -> None:
    import torch
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()


def set_ddr_flush(enabled: bool) -> None:
    """Host-visible results are made coherent by stream synchronisation on CUDA; recorded only."""
    global _flush
    _flush = bool(enabled)


def get_ddr_flush() -> bool:
    return _flush


def set_ddr_flush_force(enabled: bool) -> None:
    set_ddr_flush(enabled)


def get_ddr_flush_force() -> bool:
    """Always true in effect: every device-to-host read goes through a stream synchronisation."""
    return True


def is_available() -> bool:
    """A CUDA device is visible and the native kernel library is built."""
    import torch
    from .. import _native
    return bool(torch.cuda.is_available()) and _native.available()


def get_amp_supported_dtype() -> list:
    """Compute dtypes of the kernels (accumulation is fp32 in tensor memory either way)."""
    import torch
    return [torch.float16, torch.bfloat16]


def is_autocast_available() -> bool:
    return True


def get_spm_mode() -> bool:
    """There is no scratch-pad mode to switch: operators place their tiles in shared / tensor memory themselves."""
    return False


def get_allreduce_twostage() -> bool:
    """The fused tensor-parallel all-reduce has a two-shot (reduce-scatter + all-gather) form, which the GEMM picks by
    itself for outputs above 256 rows; there is no process-wide switch, so this reports that the form is available."""
    return True


def get_linear_acc32() -> bool:
    """Linear layers always accumulate in fp32 (tensor-memory accumulators)."""
    return True


def get_memory_stats() -> dict:
    return memory_stats()


def reset_accumulated_memory_stats() -> None:
    import torch
    if torch.cuda.is_available():
        torch.cuda.reset_accumulated_memory_stats()


def get_cross_layer_batch_prefill() -> int:
    return _cross_layer_batch


def spm_alloc_reset_temporary() -> None:
    """Release the transient scratch of the stand-alone operators (split-K workspaces)."""
    import torch
    torch.ops.rpu.spm_alloc_reset_temporary()


reset_temporary_spm = spm_alloc_reset_temporary


def reset_all_spm() -> None:
    import torch
    torch.ops.rpu.spm_alloc_reset_all()


def set_cross_layer_batch_size(n: int) -> None:
    """The whole layer loop is one CUDA graph here; the value is recorded for introspection."""
    global _cross_layer_batch
    if not isinstance(n, int) or n < 0:
        raise ValueError("cross-layer batch size must be a non-negative integer")
    _cross_layer_batch = n


def set_cross_layer_batch_prefill(n: int) -> None:
    set_cross_layer_batch_size(n)


def get_cross_layer_batch_size() -> int:
    return _cross_layer_batch


def shutdown() -> None:
    """Ordered teardown: graph caches first (they hold executable graphs), then cached memory."""
    from ..graph import GraphCache
    GraphCache.clear_all()
    empty_cache()
