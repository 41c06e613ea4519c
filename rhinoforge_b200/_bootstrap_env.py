"""What has to be arranged in the process before PyTorch is imported (standard library only at import time;
the reference does the same in ``python/rpu_backend/_bootstrap_env.py:1-33``)."""
from __future__ import annotations

import resource

WANTED_OPEN_FILES = 1 << 20


def ensure_nofile_limit(wanted: int = WANTED_OPEN_FILES) -> int:
    """Lift the soft ``RLIMIT_NOFILE`` as far as the hard limit allows and return the soft limit now in force.

    A sharded checkpoint is one memory-mapped file per shard and every CUDA-IPC peer mapping holds a descriptor, so an
    8-way tensor-parallel load of a large model runs past the usual 1024.  Failing to raise the limit is not an error."""
    soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
    goal = wanted if hard == resource.RLIM_INFINITY else min(wanted, hard)
    if soft < goal:
        try:
            resource.setrlimit(resource.RLIMIT_NOFILE, (goal, hard))
            soft = goal
        except (ValueError, OSError):
            pass
    return soft


def configure_hf_cache() -> None:
    """Point the Hugging Face cache variables at the model cache unless the user already set them."""
    from .model_registry import set_hf_home_env
    set_hf_home_env()


__all__ = ["ensure_nofile_limit", "configure_hf_cache", "WANTED_OPEN_FILES"]
