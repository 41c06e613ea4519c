"""``RPUCache``: the KV cache object users hand to ``generate`` / ``forward``.

Compatible with the Hugging Face ``Cache`` protocol as far as the fused runtime needs it
(``get_seq_length``, ``get_max_length``, ``update`` is inert, iteration over layers), backed by
the paged pool of :class:`rhinoforge_b200.runtime.kv_cache.PagedKV`.  ``position`` is the only
source of truth for the cached length; the model advances it, HF's ``update()`` never does.
``to_dynamic_cache()`` returns the dense ``[B, kv_heads, position, head_dim]`` tensors the
reference produces by un-swizzling its blocked layout
(``python/rpu_backend/api/cache.py:78-197,239-256,312-475``).
"""
from __future__ import annotations

from numbers import Integral
from typing import Optional

import torch

from ..runtime.control import rpu_env_int
from ..runtime.device import resolve_device
from ..runtime.kv_cache import PagedKV

try:  # the HF base class is optional
    from transformers.cache_utils import Cache as _HFCache
except Exception:  # noqa: BLE001
    _HFCache = object

_REQUIRED = object()


def _padding_room(model) -> int:
    """Head-room the prefill planner may use: the exact ``padding_rows`` or the budget."""
    cfg = getattr(model, "_rpu_execution", None) or {}
    stage = cfg.get("prefill", {}) if hasattr(cfg, "get") else {}
    rows = stage.get("padding_rows") if hasattr(stage, "get") else None
    if isinstance(rows, int):
        return rows
    budget = stage.get("padding_budget") if hasattr(stage, "get") else None
    if isinstance(budget, int):
        return budget
    return rpu_env_int("RPU_CAUSAL_PREFILL_PADDING_BUDGET", 64)


class RPUCache(PagedKV, _HFCache):
    is_sliding_window = False

    def __init__(self, num_layers: int, batch_size: int, max_seq_len: int, num_kv_heads: int, head_dim: int,
                 device="rpu", dtype: torch.dtype = torch.float16, attn_tp: int = 1):
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"RPUCache dtype must be torch.float16 or torch.bfloat16, got {dtype}")
        if isinstance(attn_tp, bool) or not isinstance(attn_tp, int) or attn_tp <= 0:
            raise ValueError(f"RPUCache attn_tp must be a positive integer, got {attn_tp!r}")
        try:
            dev = resolve_device(device) if not str(device).startswith("cpu") else torch.device("cpu")
        except (TypeError, ValueError) as exc:
            raise ValueError(f"RPUCache invalid device {device!r}") from exc
        if dev.type not in ("cpu", "cuda"):
            raise ValueError(f"RPUCache device must be cpu, rpu or cuda; got {device!r}")
        local_heads = max(1, num_kv_heads // attn_tp) if num_kv_heads >= attn_tp else 1
        PagedKV.__init__(self, num_layers, batch_size, max_seq_len, local_heads, head_dim, device=dev, dtype=dtype)
        self.total_kv_heads = num_kv_heads
        self.attn_tp = attn_tp
        self._seen_tokens = 0
        self.layers = []

    # -- the single length source ------------------------------------------------------------
    @property
    def position(self) -> int:
        return self.lengths[0]

    @position.setter
    def position(self, v: int) -> None:
        for s in range(self.batch_size):
            self.lengths[s] = int(v)

    def update_position(self, seq_len: int) -> None:
        if isinstance(seq_len, bool) or not isinstance(seq_len, Integral):
            raise ValueError(f"RPUCache seq_len must be a non-negative integer, got {seq_len!r}")
        seq_len = int(seq_len)
        if seq_len < 0 or self.position + seq_len > self.max_seq_len:
            raise ValueError(f"RPUCache position overflow: position={self.position}, seq_len={seq_len}, "
                             f"max_seq_len={self.max_seq_len}")
        self.position = self.position + seq_len
        self._seen_tokens = self.position

    def reset(self) -> None:
        self.position = 0
        self._seen_tokens = 0
        self.zero_()

    def reset_to_position(self, pos: int) -> None:
        """Rewind (or set) the length without clearing data: the prefix ``[0, pos)`` stays valid,
        the suffix is overwritten by the next forward before attention reads it."""
        if isinstance(pos, bool) or not isinstance(pos, Integral):
            raise ValueError(f"RPUCache position must be an integer in range, got {pos!r}")
        pos = int(pos)
        if not 0 <= pos <= self.max_seq_len:
            raise ValueError(f"RPUCache position must be in [0, {self.max_seq_len}], got {pos}")
        self.position = pos
        self._seen_tokens = pos

    # -- Hugging Face Cache protocol ------------------------------------------------------------
    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.position

    def get_max_length(self) -> int:
        return self.max_seq_len

    def get_max_cache_shape(self, layer_idx: int = 0) -> int:
        return self.max_seq_len

    def get_usable_length(self, new_seq_length: int, layer_idx: int = 0) -> int:
        return self.position

    def get_mask_sizes(self, cache_position, layer_idx: int = 0):
        return self.position, 0

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        """Inert: the fused runtime writes K/V pages itself."""
        return key_states, value_states

    @property
    def seen_tokens(self) -> int:
        return self._seen_tokens

    def get_cache(self, layer_idx: int):
        return self.kv[layer_idx, 0], self.kv[layer_idx, 1]

    @property
    def k_caches(self):
        return [self.kv[l, 0] for l in range(self.num_layers)]

    @property
    def v_caches(self):
        return [self.kv[l, 1] for l in range(self.num_layers)]

    def __len__(self) -> int:
        return self.num_layers

    def __getitem__(self, layer_idx: int):
        return self.get_cache(layer_idx)

    def __iter__(self):
        for i in range(self.num_layers):
            yield self.get_cache(i)

    def __repr__(self) -> str:
        return (f"RPUCache(num_layers={self.num_layers}, batch_size={self.batch_size}, "
                f"max_seq_len={self.max_seq_len}, position={self.position})")

    # -- construction from a model ----------------------------------------------------------------
    @classmethod
    def from_model(cls, model, *, input_ids=None, max_new_tokens=_REQUIRED, max_seq_len: Optional[int] = None,
                   batch_size: int = 1, device="rpu") -> "RPUCache":
        """Two mutually exclusive sizing forms:
        ``from_model(model, input_ids=ids, max_new_tokens=N)`` covers ``ids.shape[1] + N`` rows plus
        the prefill planner's padding room; ``from_model(model, max_seq_len=L)`` is explicit."""
        by_ids = input_ids is not None or max_new_tokens is not _REQUIRED
        if by_ids == (max_seq_len is not None):
            raise ValueError("RPUCache.from_model takes either (input_ids, max_new_tokens) or max_seq_len, not both")
        if by_ids:
            if input_ids is None or max_new_tokens is _REQUIRED:
                raise ValueError("RPUCache.from_model needs both input_ids and max_new_tokens")
            if isinstance(max_new_tokens, bool) or not isinstance(max_new_tokens, Integral) or max_new_tokens < 0:
                raise ValueError(f"max_new_tokens must be a non-negative integer, got {max_new_tokens!r}")
            prompt = int(input_ids.shape[-1])
            if input_ids.dim() == 2 and batch_size == 1:
                batch_size = int(input_ids.shape[0])
            need = prompt + int(max_new_tokens) + _padding_room(model) + 1
        else:
            need = int(max_seq_len)
        cfg = getattr(model, "config", None)
        text = getattr(cfg, "text_config", cfg)
        if text is None:
            raise ValueError("RPUCache.from_model: the model has no config")
        model_type = getattr(text, "model_type", "")
        if batch_size > 1 and not str(model_type).startswith(("qwen3", "llama", "gemma")):
            raise ValueError(f"RPUCache batch_size>1 is only supported for causal decoders, got {model_type!r}")
        heads = int(getattr(text, "num_key_value_heads", getattr(text, "num_attention_heads")))
        hd = int(getattr(text, "head_dim", None) or text.hidden_size // text.num_attention_heads)
        tp = getattr(model, "_rpu_tp_world", 1)
        dtype = getattr(model, "_rpu_dtype", torch.float16)
        need = (need + 15) // 16 * 16
        return cls(int(text.num_hidden_layers), batch_size, need, heads, hd, device=device, dtype=dtype, attn_tp=tp)

    def to_dynamic_cache(self):
        """Dense copy as a Hugging Face ``DynamicCache`` holding ``[B, kv_heads, position, head_dim]``."""
        from transformers.cache_utils import DynamicCache
        out = DynamicCache()
        for l in range(self.num_layers):
            ks, vs = [], []
            for b in range(self.batch_size):
                k, v = self.gather(l, b, self.position)
                ks.append(k)
                vs.append(v)
            out.update(torch.stack(ks), torch.stack(vs), l)
        return out


__all__ = ["RPUCache"]
