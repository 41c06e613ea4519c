"""Hugging Face ``generate()`` over the accelerator handle, unmodified.

:class:`HFGenerationAdapter` is a ``torch.nn.Module`` + ``transformers.GenerationMixin`` whose ``forward`` is the handle's:
``GenerationMixin.generate`` - its sampling, logits processors, stopping criteria, streamers and beam bookkeeping - then
runs as shipped, one engine launch per step.  The handle's own ``generate`` keeps the fast path (greedy decoding as one
CUDA graph per step with the arg-max on the device) and hands everything else to this adapter.

What the adapter has to supply is small: the model config and generation config, a device, the two capability
switches ``generate`` looks at, and a ``forward`` that accepts a padded batch with its attention mask at the first call
and one token per sequence afterwards.  The KV cache is the caller's ``RPUCache`` (a ``transformers.Cache`` subclass).

Reference behaviour: ``examples/causal_lm.py:60-79`` (``model.generate(**inputs, past_key_values=cache, ...)`` on the
loaded model), ``python/rpu_backend/adapters/qwen3.py:344-409`` (forward contract under ``generate``).
"""
from __future__ import annotations

from typing import Optional

import torch


def _mixin():
    from transformers import GenerationMixin
    return GenerationMixin


def make_adapter(handle):
    """Build the adapter class lazily (``transformers`` is imported only when generation is delegated)."""
    GenerationMixin = _mixin()
    from transformers import GenerationConfig

    class HFGenerationAdapter(torch.nn.Module, GenerationMixin):
        main_input_name = "input_ids"
        base_model_prefix = "model"
        _is_stateful = False
        _supports_cache_class = True
        _supports_static_cache = False
        _supports_default_dynamic_cache = staticmethod(lambda: False)

        def __init__(self, handle):
            super().__init__()
            self.handle = handle
            self.config = handle.config
            gc = getattr(handle, "generation_config", None)
            self.generation_config = gc if gc is not None else GenerationConfig.from_model_config(handle.config)
            self._anchor = torch.nn.Parameter(torch.empty(0, device=handle.device, dtype=handle.dtype), requires_grad=False)

        @property
        def device(self) -> torch.device:
            return self.handle.device

        @property
        def dtype(self) -> torch.dtype:
            return self.handle.dtype

        @classmethod
        def can_generate(cls) -> bool:
            return True

        def get_input_embeddings(self):
            return None

        def get_output_embeddings(self):
            return None

        @staticmethod
        def is_remote_code() -> bool:
            return False

        def forward(self, input_ids: Optional[torch.Tensor] = None, past_key_values=None, attention_mask: Optional[torch.Tensor] = None,
                    position_ids: Optional[torch.Tensor] = None, logits_to_keep: int = 0, use_cache: bool = True,
                    return_dict: bool = True, **kwargs):
            out = self.handle.forward(input_ids=input_ids, past_key_values=past_key_values, attention_mask=attention_mask,
                                      logits_to_keep=logits_to_keep, use_cache=use_cache, return_dict=True)
            out.logits = out.logits.to(input_ids.device)
            return out

        def _reorder_cache(self, past_key_values, beam_idx):
            raise NotImplementedError("beam search would have to re-order the paged KV pool; use sampling or greedy decoding")

    return HFGenerationAdapter(handle)


__all__ = ["make_adapter"]
