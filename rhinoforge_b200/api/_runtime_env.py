"""Policy-scoped ``runtime_env`` validation.

A policy facade lets its caller pass a few environment settings that are applied for the lifetime of that
policy only.  Each facade owns an :class:`EnvPolicy`: the keys it accepts and the keys that can only take
effect when set before the package is imported.  ``EnvPolicy.apply`` turns a caller's mapping into a plain
``{str: str}`` dict or raises ``ValueError`` with the message the reference uses for the same mistake
(``python/rpu_backend/api/_runtime_env.py:15-54``), so callers written against either package see the
same text.
"""
from __future__ import annotations

from collections.abc import Collection, Mapping
from dataclasses import dataclass, field
from typing import Dict, FrozenSet, Optional

PREIMPORT_ONLY = frozenset({"RPU_LOG_LEVEL", "RPU_MODEL_CACHE", "RF_PDL", "RF_B200_NO_BUILD"})

# characters that cannot appear in a process-environment key
_KEY_FORBIDDEN = ("=", "\0")


def _key_problem(key: object) -> bool:
    """True when ``key`` cannot name an environment variable at all."""
    return not (isinstance(key, str) and key != "" and not any(ch in key for ch in _KEY_FORBIDDEN))


@dataclass(frozen=True)
class EnvPolicy:
    """The environment keys one policy facade accepts."""

    owner: str
    allowed: FrozenSet[str]
    preimport_only: FrozenSet[str] = field(default=PREIMPORT_ONLY)

    def _classify(self, key: object) -> Optional[str]:
        """Error text for ``key`` or None when it is accepted."""
        if _key_problem(key):
            return f"{self.owner} runtime_env has invalid environment key {key!r}"
        if key in self.allowed:
            return None
        if key in self.preimport_only:
            return f"{self.owner} runtime_env key {key!r} must be set before importing rpu_backend"
        return f"{self.owner} runtime_env has unsupported environment key {key!r}"

    def _render(self, key: str, value: object) -> str:
        text = str(value)
        if "\0" in text:
            raise ValueError(f"{self.owner} runtime_env[{key!r}] contains a null byte")
        return text

    def apply(self, runtime_env: Optional[Mapping]) -> Dict[str, str]:
        if runtime_env is None:
            return {}
        if not isinstance(runtime_env, Mapping):
            raise ValueError(f"{self.owner} runtime_env must be a mapping")
        problems = [msg for msg in map(self._classify, runtime_env) if msg is not None]
        if problems:
            raise ValueError(problems[0])
        return {key: self._render(key, value) for key, value in runtime_env.items()}


def normalize_runtime_env(runtime_env: Optional[Mapping], *, owner: str, allowed: Collection[str],
                          preimport_only: Collection[str] = PREIMPORT_ONLY) -> Dict[str, str]:
    """Function form of :meth:`EnvPolicy.apply` (the call shape the policy facades use)."""
    return EnvPolicy(owner, frozenset(allowed), frozenset(preimport_only)).apply(runtime_env)


__all__ = ["EnvPolicy", "normalize_runtime_env", "PREIMPORT_ONLY"]
