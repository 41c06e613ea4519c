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
    @staticmethod
    def _unpad(ids: torch.Tensor, attention_mask):
        """Rows of a padded batch without their padding: ``(rows, keep)`` where ``keep[b]`` holds the kept column indices."""
        if attention_mask is None:
            return [ids[b] for b in range(ids.shape[0])], None
        m = torch.as_tensor(attention_mask).to("cpu").bool()
        if m.shape[-1] > ids.shape[-1]:           # a running mask of prompt + generated tokens: the new columns are the last ones
            m = m[:, -ids.shape[-1]:]
        if bool(m.all()):
            return [ids[b] for b in range(ids.shape[0])], None
        keep = []
        for b in range(ids.shape[0]):
            cols = m[b].nonzero().flatten()
            if cols.numel() == 0:
                raise RPUBackendError(f"sequence {b} is all padding")
            if int(cols[-1] - cols[0]) + 1 != cols.numel():
                raise RPUBackendError("attention masks with holes are not supported: padding must sit on one side")
            keep.append(cols)
        return [ids[b][keep[b].to(ids.device)] for b in range(ids.shape[0])], keep

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor = None, past_key_values=None, attention_mask=None,
                position_ids=None, logits_to_keep: int = 1, use_cache: bool = True, return_dict: bool = True, **kw):
        """Append ``input_ids`` at ``past_key_values.position`` and return logits ``[B, rows, vocab]``:
        ``logits_to_keep = k > 0`` the last ``k`` rows of every sequence, ``0`` every row.  A padded batch comes with its
        ``attention_mask`` (padding on one side): the padding columns are dropped before the launch - the engine packs
        sequences of unequal length - and their logits rows read zero."""
        k = 1 if logits_to_keep is None else int(logits_to_keep)
        if k < 0:
            raise RPUBackendError("logits_to_keep must be 0 (all rows) or a positive row count")
        self._bind(past_key_values)
        ids = input_ids if input_ids.dim() == 2 else input_ids[None]
        rows, keep = self._unpad(ids, attention_mask)
        start = past_key_values.position
        if k == 1:
            _, last = self.engine.extend(rows, return_logits=True)
            per_seq = [last[b:b + 1] for b in range(len(rows))]
        else:
            _, per_seq = self.engine.extend(rows, return_logits=True, logits_rows=k)
        if self.engine.tp.enabled:
            import torch.distributed as dist
            gathered = []
            for lg in per_seq:
                parts = [torch.empty_like(lg) for _ in range(self.engine.tp.world)]
                dist.all_gather(parts, lg.contiguous(), group=self.engine.tp.group)
                gathered.append(torch.cat(parts, -1))
            per_seq = gathered
        L = ids.shape[1] if k == 0 else min(k, ids.shape[1])
        if all(lg.shape[0] == L for lg in per_seq):
            logits = torch.stack(per_seq)
        else:                                       # unequal real lengths: rows sit where their columns were
            logits = per_seq[0].new_zeros((len(rows), L, per_seq[0].shape[-1]))
            first_col = ids.shape[1] - L
            for b, lg in enumerate(per_seq):
                cols = keep[b][-lg.shape[0]:] - first_col
                logits[b, cols.to(logits.device)] = lg
        # the resolved plan of this call (variable-length launches run every length as it is: no padding rows)
        from .decoder import default_chunk_resolver, plan_bounded_prefill_execution
        n_rows = int(rows[0].numel())
        exec_len, chunk = plan_bounded_prefill_execution(n_rows, max(start + n_rows, 1), 0,
                                                         default_chunk_resolver(self.engine.max_tokens), start)
        self._rpu_last_execution_plan = {"stage": "prefill" if n_rows > 1 else "decode", "logical_len": n_rows,
                                         "execution_len": exec_len, "chunk_size": chunk,
                                         "padding_rows": exec_len - n_rows, "position": start}
        if not return_dict:
            return (logits, past_key_values)
        from transformers.modeling_outputs import CausalLMOutputWithPast
        return CausalLMOutputWithPast(logits=logits, past_key_values=past_key_values)

    __call__ = forward

    # -- generation --------------------------------------------------------------------------------
    @property
    def hf(self):
        """This handle as a ``transformers.GenerationMixin`` model: ``model.hf.generate(...)`` is Hugging Face's own loop."""
        if getattr(self, "_hf_adapter", None) is None:
            from .hf_generation import make_adapter
            self._hf_adapter = make_adapter(self)
        return self._hf_adapter

    _FAST_KWARGS = frozenset({"use_cache", "pad_token_id", "return_dict_in_generate", "num_beams", "temperature", "top_k", "top_p"})

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, past_key_values=None, max_new_tokens: Optional[int] = None,
                 do_sample: bool = False, attention_mask=None, eos_token_id=None, **kw) -> torch.Tensor:
        """``[B, prompt + new]`` token ids on the input's device, like Hugging Face ``generate``.

        Greedy decoding of equal-length prompts runs on the fast path: the whole decode step, arg-max included, is one CUDA
        graph and tokens never visit the host (generation stops early only when every sequence has produced
        ``eos_token_id``, checked once per 16 steps).  Anything else - sampling, logits processors, stopping criteria,
        streamers, a padded batch, ``max_length`` - is Hugging Face's unmodified ``GenerationMixin.generate`` driving this
        handle's ``forward`` (:attr:`hf`)."""
        ids2 = input_ids if input_ids.dim() == 2 else input_ids[None]
        padded = attention_mask is not None and not bool(torch.as_tensor(attention_mask).bool().all())
        plain = (not do_sample and not padded and max_new_tokens is not None and set(kw) <= self._FAST_KWARGS
                 and kw.get("num_beams", 1) == 1 and not kw.get("return_dict_in_generate", False))
        if not plain:
            if past_key_values is None:
                from ..api.cache import RPUCache
                budget = max_new_tokens if max_new_tokens is not None else max(int(kw.get("max_length", 0)) - ids2.shape[1], 1)
                past_key_values = RPUCache.from_model(self, input_ids=ids2, max_new_tokens=budget)
            extra = dict(kw)
            if max_new_tokens is not None:
                extra["max_new_tokens"] = max_new_tokens
            if eos_token_id is not None:
                extra["eos_token_id"] = eos_token_id
            out = self.hf.generate(input_ids=ids2, attention_mask=attention_mask, past_key_values=past_key_values,
                                   do_sample=do_sample, use_cache=True, **extra)
            self.engine.check_status()
            return out
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
