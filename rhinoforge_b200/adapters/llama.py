"""Llama causal-LM adapter: the Llama-3.2-1B profile (no QK-norm, head_dim 64, tied embeddings).
Reference: ``python/rpu_backend/adapters/llama.py``."""
from .causal_base import CausalLMAdapter


class LlamaAdapter(CausalLMAdapter):
    ARCH = "LlamaForCausalLM"
    FAMILY = "Llama"
    SUPPORTED_PROFILES = frozenset({(2048, 8192, 16, 8)})
    UNLISTED_GATE = "RPU_LLAMA_ALLOW_UNLISTED_PROFILE"


__all__ = ["LlamaAdapter"]
