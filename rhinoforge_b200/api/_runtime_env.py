"""Validation of policy-scoped ``runtime_env`` mappings: a policy facade accepts only its own allow-listed
environment keys, as strings, and names the keys that must be set before the package is imported
(reference: ``python/rpu_backend/api/_runtime_env.py:15-54``)."""
from __future__ import annotations

from collections.abc import Collection, Mapping
from typing import Dict, Optional

PREIMPORT_ONLY = frozenset({"RPU_LOG_LEVEL", "RPU_MODEL_CACHE", "RF_PDL", "RF_B200_NO_BUILD"})


def normalize_runtime_env(runtime_env: Optional[Mapping], *, owner: str, allowed: Collection[str],
                          preimport_only: Collection[str] = PREIMPORT_ONLY) -> Dict[str, str]:
    if runtime_env is None:
        return {}
    if not isinstance(runtime_env, Mapping):
        raise ValueError(f"{owner} runtime_env must be a mapping")
    out: Dict[str, str] = {}
    for key, value in runtime_env.items():
        if not isinstance(key, str) or not key or "=" in key or "\0" in key:
            raise ValueError(f"{owner} runtime_env has invalid environment key {key!r}")
        if key not in allowed:
            if key in preimport_only:
                raise ValueError(f"{owner} runtime_env key {key!r} must be set before importing rpu_backend")
            raise ValueError(f"{owner} runtime_env has unsupported environment key {key!r}")
        text = str(value)
        if "\0" in text:
            raise ValueError(f"{owner} runtime_env[{key!r}] contains a null byte")
        out[key] = text
    return out


__all__ = ["normalize_runtime_env", "PREIMPORT_ONLY"]
