"""A fill-in adapter for a decoder-only language model (reference counterpart:
``python/rpu_backend/adapters/_template/minimal_causal_lm.py:83-317``; the flow is that of ``adapters/qwen3.py`` and
``adapters/llama.py`` here).

What a causal-LM adapter has to decide, in the order the questions come up:

1. **Which checkpoints are admitted.**  Admission is deny-by-default on the tuple ``(hidden_size, intermediate_size,
   num_hidden_layers, num_key_value_heads)``: list the shapes you ran the numerics test on in ``SUPPORTED_PROFILES``
   (``W8A16_ONLY_PROFILES`` for shapes that only fit quantised).  ``UNLISTED_GATE`` names an environment variable that
   admits any shape for evaluation when set to the literal ``1``.
2. **How the Hugging Face config maps onto the native stack.**  ``DecoderConfig.from_hf`` reads the usual fields
   (RMSNorm eps, rope theta and scaling, QK-norm, tied embeddings, head_dim).  Override ``decoder_config`` only for what
   it cannot know - a sliding window, a partial rotary dimension, a different activation.
3. **How checkpoint tensor names map onto the decoder's weight set.**  The engine asks for Hugging Face Llama-style names
   (``model.layers.{i}.self_attn.q_proj.weight`` ...).  If the family names things differently, override ``_weights``
   and translate in the getter - never rename tensors on disk.
4. **Which execution knobs the family honours.**  ``SUPPORTED_EXECUTION`` lists the ``rpu_execution`` stages and fields;
   a request outside it is refused before any weight is read.

Nothing else is per-family: weight packing, the KV pool, graphs, tensor parallelism and the ``generate`` / ``forward``
surface come from ``CausalLMAdapter.to_rpu`` and ``RPUCausalLM``.

The class below is deliberately unusable until the three placeholders are replaced, so that a half-edited copy fails
with one clear message instead of registering under a nonsense architecture name.
"""
from __future__ import annotations

from typing import Callable

import torch

from ...api.errors import RPUBackendError
from ...models.decoder import DecoderConfig
from ..causal_base import CausalLMAdapter

_PLACEHOLDER_ARCH = "<YourArch>ForCausalLM"
_PLACEHOLDER_FAMILY = "<YourFamily>"


class TemplateNotFilledError(RPUBackendError):
    """The template was used without replacing its placeholders."""


class MinimalCausalLMAdapter(CausalLMAdapter):
    # -- 1. identity and admission ----------------------------------------------------------------------------------
    ARCH = _PLACEHOLDER_ARCH                    # the string in config.json["architectures"][0]
    FAMILY = _PLACEHOLDER_FAMILY                # used in messages only
    SUPPORTED_PROFILES = frozenset({
        # (hidden_size, intermediate_size, num_hidden_layers, num_key_value_heads), one row per validated checkpoint:
        # (2048, 8192, 16, 8),
    })
    W8A16_ONLY_PROFILES = frozenset()
    UNLISTED_GATE = ""                          # e.g. "RPU_<FAMILY>_ALLOW_UNLISTED_PROFILE"

    # -- 4. execution knobs -----------------------------------------------------------------------------------------
    SUPPORTED_EXECUTION = {"prefill": ("chunk_size", "padding_rows", "padding_budget")}

    @classmethod
    def check_template_filled(cls) -> None:
        left = [what for what, unfilled in (
            ("ARCH", cls.ARCH == _PLACEHOLDER_ARCH or not cls.ARCH),
            ("FAMILY", cls.FAMILY == _PLACEHOLDER_FAMILY or not cls.FAMILY),
            ("SUPPORTED_PROFILES (or W8A16_ONLY_PROFILES / UNLISTED_GATE)",
             not (cls.SUPPORTED_PROFILES or cls.W8A16_ONLY_PROFILES or cls.UNLISTED_GATE)),
        ) if unfilled]
        if left:
            raise TemplateNotFilledError(f"{cls.__name__}: the adapter template still has placeholders: {', '.join(left)}")

    @classmethod
    def preflight(cls, config) -> None:
        cls.check_template_filled()
        super().preflight(config)
        # family-specific refusals that can be decided from the config alone go here, for example:
        #   if getattr(config, "attention_bias", False): raise UnsupportedModelError("... QKV bias not validated")

    def __init__(self, *args, **kwargs):
        self.check_template_filled()
        super().__init__(*args, **kwargs)

    # -- 2. config mapping ------------------------------------------------------------------------------------------
    def decoder_config(self) -> DecoderConfig:
        cfg = DecoderConfig.from_hf(self.config)
        # adjust what from_hf cannot infer, e.g.  cfg = dataclasses.replace(cfg, qk_norm=False)
        return cfg

    # -- 3. weight names --------------------------------------------------------------------------------------------
    #: checkpoint-name prefix -> the Llama-style prefix the decoder asks for; the default maps nothing
    RENAMES = ()

    def _weights(self) -> Callable[[str], torch.Tensor]:
        get = super()._weights()
        if not self.RENAMES:
            return get

        def to_checkpoint(name: str) -> str:
            for theirs, ours in self.RENAMES:
                if name.startswith(ours):
                    return theirs + name[len(ours):]
            return name

        def from_checkpoint(name: str) -> str:
            for theirs, ours in self.RENAMES:
                if name.startswith(theirs):
                    return ours + name[len(theirs):]
            return name

        def renamed(name: str) -> torch.Tensor:
            return get(to_checkpoint(name))

        names = getattr(get, "names", None)
        if names is not None:
            renamed.names = frozenset(from_checkpoint(n) for n in names)  # type: ignore[attr-defined]
        scale = getattr(get, "scale", None)
        if scale is not None:
            renamed.scale = lambda n: scale(to_checkpoint(n))  # type: ignore[attr-defined]
        return renamed


def register(adapter_cls=MinimalCausalLMAdapter) -> None:
    """Bind ``adapter_cls.ARCH`` in the adapter registry (what a plug-in's entry point calls)."""
    from ...runtime.registry import register_adapter
    adapter_cls.check_template_filled()
    register_adapter(adapter_cls.ARCH, adapter_cls)


__all__ = ["MinimalCausalLMAdapter", "TemplateNotFilledError", "register"]
