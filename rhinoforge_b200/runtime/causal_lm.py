"""Runtime handle of a causal LM that has been moved to the accelerator.

``RPUCausalLM`` is what ``RPUModelForCausalLM.from_pretrained(..., device="rpu")`` and
``model.to("rpu")`` return: an object with the call shapes users of the Hugging Face model rely
on -- ``generate(ids, past_key_values=cache, max_new_tokens=n, do_sample=False)`` and
``model(input_ids=..., past_key_values=cache, logits_to_keep=1, use_cache=True)`` -- served by
:class:`rhinoforge_b200.runtime.engine.DecoderEngine`.  Moving it back to the CPU is refused:
the weight transform happens exactly once (reference contract:
``python/rpu_backend/adapters/qwen3.py:344-409``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..graph.lazy_init_guard import mark_install_checked, verify_lazy_init
from .errors import RPUBackendError
from .engine import DecoderEngine


class RPUCausalLM:
    def __init__(self, engine: DecoderEngine, hf_config, *, execution=None, owner=None):
        self.engine = engine
        self.config = hf_config
        self._rpu_execution = execution
        self._rpu_is_ready = True
        self._rpu_dtype = engine.dtype
        self._rpu_tp_world = engine.tp.world
        self._owner = owner
        self._rpu_last_execution_plan = None
        self.generation_config = getattr(owner, "generation_config", None)
        # everything the decode path reads exists from here on; nothing is created at the first forward
        mark_install_checked(self, ("engine", "_rpu_execution", "_rpu_dtype", "_rpu_tp_world"))
        verify_lazy_init(self)

    # -- module-like surface --------------------------------------------------------------------
    @property
    def device(self) -> torch.device:
        return self.engine.device

    @property
    def dtype(self) -> torch.dtype:
        return self.engine.dtype

    def eval(self):
        return self

    def to(self, device=None, *a, **kw):
        name = str(device).lower() if device is not None else ""
        if name.startswith(("rpu", "cuda")) or device is None:
            return self
        raise RPUBackendError("this model's weights were packed for the accelerator exactly once; "
                              "it cannot be moved back to the CPU -- reload the checkpoint instead")

    def cpu(self):
        return self.to("cpu")

    # -- helpers ----------------------------------------------------------------------------------
    def _bind(self, cache) -> None:
        if cache is None:
            raise RPUBackendError("pass past_key_values=RPUCache.from_model(model, ...)")
        self.engine.bind_cache(cache)

    def _rows(self, input_ids: torch.Tensor):
        ids = input_ids if input_ids.dim() == 2 else input_ids[None]
        return [ids[b] for b in range(ids.shape[0])]

    # -- forward -----------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor = None, past_key_values=None, attention_mask=None,
                position_ids=None, logits_to_keep: int = 1, use_cache: bool = True, return_dict: bool = True, **kw):
        """Append ``input_ids`` at ``past_key_values.position`` and return the logits of the last
        row of every sequence (``logits_to_keep`` must be 1: the fused head runs on one row per
        sequence).  An all-ones ``attention_mask`` is accepted; padding masks are not."""
        if logits_to_keep not in (1, None):
            raise RPUBackendError("the fused lm_head returns one row per sequence: pass logits_to_keep=1")
        if attention_mask is not None and not bool(torch.as_tensor(attention_mask).bool().all()):
            raise RPUBackendError("only all-ones attention masks are supported (equal real lengths)")
        self._bind(past_key_values)
        rows = self._rows(input_ids)
        start = past_key_values.position
        _, logits = self.engine.extend(rows, return_logits=True)
        if self.engine.tp.enabled:
            import torch.distributed as dist
            parts = [torch.empty_like(logits) for _ in range(self.engine.tp.world)]
            dist.all_gather(parts, logits, group=self.engine.tp.group)
            logits = torch.cat(parts, -1)
        # the resolved plan of this call (variable-length launches run every length as it is: no padding rows)
        from .decoder import default_chunk_resolver, plan_bounded_prefill_execution
        n_rows = int(rows[0].numel())
        exec_len, chunk = plan_bounded_prefill_execution(n_rows, max(start + n_rows, 1), 0,
                                                         default_chunk_resolver(self.engine.max_tokens), start)
        self._rpu_last_execution_plan = {"stage": "prefill" if n_rows > 1 else "decode", "logical_len": n_rows,
                                         "execution_len": exec_len, "chunk_size": chunk,
                                         "padding_rows": exec_len - n_rows, "position": start}
        logits = logits[:, None, :]
        if not return_dict:
            return (logits, past_key_values)
        from transformers.modeling_outputs import CausalLMOutputWithPast
        return CausalLMOutputWithPast(logits=logits, past_key_values=past_key_values)

    __call__ = forward

    # -- generation --------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, past_key_values=None, max_new_tokens: Optional[int] = None,
                 do_sample: bool = False, attention_mask=None, eos_token_id=None, **kw) -> torch.Tensor:
        """Greedy generation.  Returns ``[B, prompt + new]`` token ids on the input's device, like
        Hugging Face ``generate``.  ``do_sample`` must be False; generation stops early only when
        every sequence has produced ``eos_token_id`` (checked once per 16 steps)."""
        if do_sample:
            raise RPUBackendError("sampling is not supported: pass do_sample=False")
        if max_new_tokens is None or max_new_tokens < 1:
            raise RPUBackendError("max_new_tokens must be a positive integer")
        ids = input_ids if input_ids.dim() == 2 else input_ids[None]
        if past_key_values is None:
            from ..api.cache import RPUCache
            past_key_values = RPUCache.from_model(self, input_ids=ids, max_new_tokens=max_new_tokens)
        self._bind(past_key_values)
        rows = self._rows(ids)
        first = self.engine.extend(rows)
        new = [first[:, None]]
        remaining = max_new_tokens - 1
        eos = None if eos_token_id is None else torch.as_tensor(eos_token_id, device=self.engine.device).flatten()
        done = torch.zeros(len(rows), dtype=torch.bool, device=self.engine.device)
        while remaining > 0:
            n = min(remaining, 16) if eos is not None else remaining
            toks = self.engine.decode(n).clone()
            new.append(toks)
            remaining -= n
            if eos is not None:
                done |= torch.isin(torch.cat(new, 1), eos).any(1)
                if bool(done.all()):
                    break
        # the last produced token has not been fed back: the cache holds prompt + new - 1 rows
        self.engine.check_status()
        out = torch.cat([ids.to(self.engine.device, torch.int64), torch.cat(new, 1).to(torch.int64)], 1)
        return out.to(input_ids.device)

    def close(self) -> None:
        self.engine.close()
