"""Qwen3 causal-LM adapter.

Admitted profiles ``(hidden, intermediate, layers, kv_heads)``: 0.6B, 1.7B, 4B, 8B in fp16/bf16;
14B and 32B only as W8A16 checkpoints with an untied int8 lm_head and fp16 embeddings (the 32B
profile is the tensor-parallel target; the reference stops at 14B:
``python/rpu_backend/adapters/qwen3.py:119-132,158-191``).  Everything else is denied by default;
``RPU_QWEN3_ALLOW_UNLISTED_PROFILE=1`` admits an unlisted shape for evaluation.
"""
from .causal_base import CausalLMAdapter


class Qwen3Adapter(CausalLMAdapter):
    ARCH = "Qwen3ForCausalLM"
    FAMILY = "Qwen3"
    SUPPORTED_PROFILES = frozenset({
        (1024, 3072, 28, 8),
        (2048, 6144, 28, 8),
        (2560, 9728, 36, 8),
        (4096, 12288, 36, 8),
    })
    W8A16_ONLY_PROFILES = frozenset({
        (5120, 17408, 40, 8),
        (5120, 25600, 64, 8),
    })
    UNLISTED_GATE = "RPU_QWEN3_ALLOW_UNLISTED_PROFILE"
    # certified context envelope per profile (tokens); bounded by device memory, not by scratch-pad
    MAX_KV = {(1024, 3072, 28, 8): 40960, (2048, 6144, 28, 8): 40960, (2560, 9728, 36, 8): 40960,
              (4096, 12288, 36, 8): 40960, (5120, 17408, 40, 8): 40960, (5120, 25600, 64, 8): 40960}


__all__ = ["Qwen3Adapter"]
