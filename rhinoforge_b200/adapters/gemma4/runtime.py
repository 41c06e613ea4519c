"""Gemma4 adapter: a Hugging Face Gemma4 model (text-only or the text tower of the multimodal wrapper) or its
checkpoint tensors -> :class:`Gemma4Handle` over :class:`rhinoforge_b200.models.gemma4.Gemma4Engine`.

    handle = Gemma4Adapter(hf_model).to_rpu(max_seq_len=4096)
    out = handle.generate(input_ids, max_new_tokens=32)            # [B, prompt + new], greedy
    logits = handle(input_ids).logits                              # [B, rows, vocab] fp32

Admission is config-only and fail-closed (mixture-of-experts blocks, other activations and bidirectional attention are
rejected before a weight is read).  Reference: ``src/fused/rpu_gemma4_model.cpp:1-24`` (what the decoder runs),
``python/rpu_backend/adapters/gemma4/geometry.py`` (per-layer table shared with the cache plan).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ...models.gemma4 import Gemma4Engine, preflight
from ...runtime.errors import RPUBackendError, UnsupportedModelError


def _text(config):
    return getattr(config, "text_config", config)


class Gemma4Handle:
    def __init__(self, engine: Gemma4Engine, config):
        self.engine, self.config = engine, config

    @property
    def device(self) -> torch.device:
        return self.engine.device

    @property
    def dtype(self) -> torch.dtype:
        return self.engine.dtype

    def eval(self):
        return self

    def to(self, device=None, *a, **kw):
        if device is None or str(device).lower().startswith(("rpu", "cuda")):
            return self
        raise RPUBackendError("this model's weights were packed for the accelerator exactly once; reload the checkpoint instead")

    @staticmethod
    def _rows(input_ids: torch.Tensor, attention_mask=None):
        ids = input_ids if input_ids.dim() == 2 else input_ids[None]
        if attention_mask is None:
            return [ids[b] for b in range(ids.shape[0])]
        m = torch.as_tensor(attention_mask).bool().cpu()
        return [ids[b][m[b].to(ids.device)] for b in range(ids.shape[0])]

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, attention_mask=None, past_key_values=None, logits_to_keep: int = 0, **kw):
        """Starts from an empty cache unless ``past_key_values`` is this handle (continue the sequences it holds)."""
        from transformers.modeling_outputs import CausalLMOutputWithPast
        rows = self._rows(input_ids, attention_mask)
        if past_key_values is not self:
            self.engine.reset()
        if logits_to_keep == 1:
            logits = self.engine.extend(rows)[:, None, :]
        else:
            per = self.engine.extend(rows, all_logits=True)
            keep = max(r.shape[0] for r in per) if not logits_to_keep else logits_to_keep
            if any(r.shape[0] < keep for r in per) and len({r.shape[0] for r in per}) > 1:
                raise RPUBackendError("sequences of unequal length return their rows only with logits_to_keep=1")
            logits = torch.stack([r[-keep:] for r in per])
        return CausalLMOutputWithPast(logits=logits, past_key_values=self)

    __call__ = forward

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, attention_mask=None, do_sample: bool = False, **kw) -> torch.Tensor:
        if do_sample:
            raise RPUBackendError("this handle decodes greedily: pass do_sample=False")
        rows = self._rows(input_ids, attention_mask)
        if len({int(r.numel()) for r in rows}) > 1:
            raise RPUBackendError("generate() returns a rectangular tensor: pass sequences of one length (use the engine for ragged batches)")
        new = self.engine.generate(rows, max_new_tokens)
        ids = input_ids if input_ids.dim() == 2 else input_ids[None]
        return torch.cat((ids.to(new.device, torch.int64), new.to(torch.int64)), 1).to(input_ids.device)

    def close(self) -> None:
        self.engine.close()


class Gemma4Adapter:
    ARCHITECTURES = ("Gemma4ForCausalLM", "Gemma4ForConditionalGeneration")

    @classmethod
    def preflight(cls, config) -> None:
        preflight(_text(config))

    def __init__(self, model=None, *, config=None, get_weight: Optional[Callable[[str], torch.Tensor]] = None, dtype=torch.bfloat16):
        if model is None and (config is None or get_weight is None):
            raise RPUBackendError("Gemma4Adapter needs a model, or a config and a weight getter")
        self.model, self.config, self._get, self.dtype = model, config if config is not None else model.config, get_weight, dtype
        self.preflight(self.config)

    def _weights(self):
        if self._get is not None:
            get, names = self._get, getattr(self._get, "names", None)
        else:
            sd = self.model.state_dict()
            get, names = (lambda n: sd[n]), set(sd)
        nested = names is not None and any(n.startswith("model.language_model.") for n in names)
        return get, ("model.language_model." if nested else "model.")

    def to_rpu(self, *, max_seq_len: int = 4096, max_batch: int = 1, max_prefill_tokens: Optional[int] = None) -> Gemma4Handle:
        get, prefix = self._weights()
        eng = Gemma4Engine(_text(self.config), get, prefix=prefix, max_seq_len=max_seq_len, max_batch=max_batch,
                           max_tokens=max_prefill_tokens or max_seq_len, dtype=self.dtype)
        self.model = None
        return Gemma4Handle(eng, self.config)


__all__ = ["Gemma4Adapter", "Gemma4Handle"]
