"""Runtime handle of a vision-language model on the accelerator.

``RPUConditionalGeneration`` serves the call shape of the Hugging Face Qwen3-VL model used by a
manual greedy loop::

    o = model(input_ids=ids, past_key_values=cache, logits_to_keep=1, use_cache=True, return_dict=True,
              attention_mask=..., pixel_values=..., image_grid_thw=..., mm_token_type_ids=...)
    o = model(input_ids=next_id, past_key_values=cache, logits_to_keep=1, use_cache=True, return_dict=True)

The first call runs the vision tower, splices image rows, computes the three-axis positions and
prefills the text decoder with DeepStack; later calls append text rows at the cache position.
``model.model.language_model`` is the object ``RPUCache.from_model`` sizes the cache from.
Reference: ``python/rpu_backend/api/conditional_generation.py:58-170``, ``examples/qwen3_vl.py:71-121``.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Optional

import torch

from .errors import RPUBackendError


class _LanguageModelView:
    """What ``RPUCache.from_model`` needs: the text config and the engine behind it."""

    def __init__(self, engine, text_config):
        self.engine, self.config = engine, text_config
        self._rpu_is_ready = True
        self._rpu_dtype = engine.dtype
        self._rpu_tp_world = engine.tp.world

    @property
    def device(self):
        return self.engine.device

    @property
    def dtype(self):
        return self.engine.dtype


class RPUConditionalGeneration:
    def __init__(self, vl_engine, hf_config, *, execution=None):
        self.vl = vl_engine
        self.config = hf_config
        self._rpu_execution = execution
        self._rpu_is_ready = True
        text_cfg = getattr(hf_config, "text_config", hf_config)
        self.model = SimpleNamespace(language_model=_LanguageModelView(vl_engine.text, text_cfg), visual=vl_engine.vision)
        self.rope_deltas = None

    @property
    def device(self) -> torch.device:
        return self.vl.device

    @property
    def dtype(self) -> torch.dtype:
        return self.vl.dtype

    def eval(self):
        return self

    def to(self, device=None, *a, **kw):
        name = str(device).lower() if device is not None else ""
        if device is None or name.startswith(("rpu", "cuda")):
            return self
        raise RPUBackendError("this model's weights were packed for the accelerator exactly once; "
                              "it cannot be moved back to the CPU -- reload the checkpoint instead")

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor = None, past_key_values=None, attention_mask=None, pixel_values=None,
                image_grid_thw=None, mm_token_type_ids=None, logits_to_keep: int = 1, use_cache: bool = True,
                return_dict: bool = True, pixel_values_videos=None, video_grid_thw=None, **kw):
        if logits_to_keep not in (1, None):
            raise RPUBackendError("the fused lm_head returns one row per sequence: pass logits_to_keep=1")
        if pixel_values_videos is not None or video_grid_thw is not None:
            raise RPUBackendError("video inputs are not supported")
        if past_key_values is None:
            raise RPUBackendError("pass past_key_values=RPUCache.from_model(model.model.language_model, ...)")
        ids = input_ids if input_ids.dim() == 2 else input_ids[None]
        if ids.shape[0] != 1:
            raise RPUBackendError("vision-language generation runs one sequence at a time")
        if attention_mask is not None and not bool(torch.as_tensor(attention_mask).bool().all()):
            raise RPUBackendError("only all-ones attention masks are supported")
        self.vl.text.bind_cache(past_key_values)
        if past_key_values.position == 0:
            _, logits = self.vl.prefill(ids[0], pixel_values, image_grid_thw, return_logits=True)
            self.rope_deltas = torch.tensor([[self.vl._next_pos - ids.shape[1]]])
        else:
            _, logits = self.vl.extend(ids[0], pixel_values, image_grid_thw, return_logits=True)
        eng = self.vl.text
        if eng.tp.enabled:
            import torch.distributed as dist
            parts = [torch.empty_like(logits) for _ in range(eng.tp.world)]
            dist.all_gather(parts, logits, group=eng.tp.group)
            logits = torch.cat(parts, -1)
        logits = logits[:, None, :]
        if not return_dict:
            return (logits, past_key_values)
        from transformers.modeling_outputs import CausalLMOutputWithPast
        return CausalLMOutputWithPast(logits=logits, past_key_values=past_key_values)

    __call__ = forward

    @torch.no_grad()
    def generate(self, input_ids, past_key_values=None, max_new_tokens: Optional[int] = None, do_sample: bool = False,
                 pixel_values=None, image_grid_thw=None, **kw) -> torch.Tensor:
        if do_sample:
            raise RPUBackendError("sampling is not supported: pass do_sample=False")
        if not max_new_tokens or max_new_tokens < 1:
            raise RPUBackendError("max_new_tokens must be a positive integer")
        ids = input_ids if input_ids.dim() == 2 else input_ids[None]
        if past_key_values is not None:
            self.vl.text.bind_cache(past_key_values)
        new = self.vl.generate(ids[0], pixel_values, image_grid_thw, max_new_tokens=max_new_tokens)
        out = torch.cat((ids.to(self.device, torch.int64), new.to(torch.int64)), 1)
        return out.to(input_ids.device)

    def close(self) -> None:
        self.vl.close()
