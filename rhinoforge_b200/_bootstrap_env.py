"""Process-environment set-up that must happen before PyTorch is imported.

Only the standard library is imported at module load (reference behaviour:
``python/rpu_backend/_bootstrap_env.py:1-33``).
"""
from __future__ import annotations

import resource

_TARGET_NOFILE = 1_048_576


def ensure_nofile_limit() -> None:
    """Raise the soft open-file limit towards the hard limit; silent, best effort.

    Sharded checkpoints are memory-mapped one file per shard and CUDA IPC keeps one
    descriptor per peer mapping, so large tensor-parallel loads can exceed 1024."""
    soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
    if soft >= _TARGET_NOFILE:
        return
    try:
        resource.setrlimit(resource.RLIMIT_NOFILE, (min(_TARGET_NOFILE, hard), hard))
    except (ValueError, OSError):
        return


def configure_hf_cache() -> None:
    from . import model_registry
    model_registry.set_hf_home_env()


__all__ = ["configure_hf_cache", "ensure_nofile_limit"]
