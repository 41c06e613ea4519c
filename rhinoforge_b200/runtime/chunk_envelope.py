"""``ChunkEnvelope``: the (maximum KV length, prefill chunk size) pair a model handle was planned for
(reference: ``python/rpu_backend/runtime/chunk_envelope.py:11-51``).  The arena and the KV pool are sized from
it once; a request outside the envelope is rejected before anything is launched."""
from __future__ import annotations

from dataclasses import dataclass

PAGE = 16


@dataclass(frozen=True)
class ChunkEnvelope:
    max_kv_len: int
    chunk: int

    def __post_init__(self):
        for name in ("max_kv_len", "chunk"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ValueError(f"ChunkEnvelope.{name} must be a positive integer, got {v!r}")
        if self.chunk % PAGE:
            raise ValueError(f"ChunkEnvelope.chunk must be a multiple of {PAGE}, got {self.chunk}")

    @property
    def pages(self) -> int:
        return (self.max_kv_len + PAGE - 1) // PAGE

    def chunks_for(self, tokens: int) -> int:
        return (tokens + self.chunk - 1) // self.chunk

    def admits(self, position: int, new_tokens: int) -> bool:
        return position >= 0 and new_tokens >= 0 and position + new_tokens <= self.max_kv_len

    def check(self, position: int, new_tokens: int) -> None:
        if not self.admits(position, new_tokens):
            raise ValueError(f"request (position={position}, new_tokens={new_tokens}) exceeds the planned envelope "
                             f"max_kv_len={self.max_kv_len}")


__all__ = ["ChunkEnvelope"]
