"""Starting point for a new decoder-only family: copy ``minimal_causal_lm.py`` to ``adapters/<family>.py``, fill the
placeholders, add a row to ``adapters/_manifest.py`` (reference counterpart: ``python/rpu_backend/adapters/_template/``)."""
from .minimal_causal_lm import MinimalCausalLMAdapter, TemplateNotFilledError, register

__all__ = ["MinimalCausalLMAdapter", "TemplateNotFilledError", "register"]
