"""``Qwen3_5Cache``: KV pages for the full-attention layers plus, for every Gated-DeltaNet layer, the
recurrent state ``[batch, Hv, Dk, Dv]`` (fp32) and the depthwise-conv state ``[batch, K-1, conv_dim]``.

    cache = Qwen3_5Cache.from_config(text_config, max_seq_len=L)

Unlike K/V pages, a recurrent state summarises the whole prefix and cannot be truncated: rewinding
to a non-zero position is refused; ``reset()`` zeroes the states and returns to position 0.
Reference: ``python/rpu_backend/api/qwen3_5_cache.py:40-204``.
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from .cache import RPUCache


class Qwen3_5Cache(RPUCache):
    def __init__(self, text_config, *, max_seq_len: int, batch_size: int = 1, device="rpu",
                 dtype: torch.dtype = torch.float16, attn_tp: int = 1):
        types = list(getattr(text_config, "layer_types"))
        self.layer_types = types
        self.full_layers = [i for i, t in enumerate(types) if t == "full_attention"]
        self.linear_layers = [i for i, t in enumerate(types) if t == "linear_attention"]
        if not self.full_layers:
            raise ValueError("Qwen3_5Cache: the configuration has no full-attention layer")
        hd = int(getattr(text_config, "head_dim", None) or text_config.hidden_size // text_config.num_attention_heads)
        if isinstance(max_seq_len, bool) or not isinstance(max_seq_len, int) or max_seq_len <= 0:
            raise ValueError(f"Qwen3_5Cache max_seq_len must be a positive integer, got {max_seq_len!r}")
        super().__init__(len(self.full_layers), batch_size, (max_seq_len + 15) // 16 * 16,
                         int(text_config.num_key_value_heads), hd, device=device, dtype=dtype, attn_tp=attn_tp)
        Hk, Hv = int(text_config.linear_num_key_heads), int(text_config.linear_num_value_heads)
        if Hk % attn_tp or Hv % attn_tp:
            raise ValueError(f"Qwen3_5Cache: linear-attention heads ({Hk}, {Hv}) do not split over attn_tp={attn_tp}")
        Hk, Hv = Hk // attn_tp, Hv // attn_tp
        Dk, Dv = int(text_config.linear_key_head_dim), int(text_config.linear_value_head_dim)
        Kc = int(getattr(text_config, "linear_conv_kernel_dim", 4))
        conv_dim = 2 * Hk * Dk + Hv * Dv
        self.conv_states: List[torch.Tensor] = [torch.zeros((batch_size, Kc - 1, conv_dim), dtype=dtype, device=self.device)
                                                for _ in self.linear_layers]
        self.recurrent_states: List[torch.Tensor] = [torch.zeros((batch_size, Hv, Dk, Dv), dtype=torch.float32,
                                                                 device=self.device) for _ in self.linear_layers]

    @classmethod
    def from_config(cls, text_config, *, max_seq_len: int, batch_size: int = 1, device="rpu",
                    dtype: torch.dtype = torch.float16, attn_tp: int = 1) -> "Qwen3_5Cache":
        text_config = getattr(text_config, "text_config", text_config)
        return cls(text_config, max_seq_len=max_seq_len, batch_size=batch_size, device=device, dtype=dtype, attn_tp=attn_tp)

    def linear_states(self, i: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(conv state, recurrent state) of the i-th linear-attention layer."""
        return self.conv_states[i], self.recurrent_states[i]

    def has_previous_state(self, layer_idx: int = 0) -> bool:
        return self.position > 0

    def reset(self) -> None:
        super().reset()
        for t in self.conv_states + self.recurrent_states:
            t.zero_()

    def reset_to_position(self, pos: int) -> None:
        if pos != 0:
            raise ValueError("Qwen3_5Cache cannot rewind to a non-zero position: recurrent states summarise the whole "
                             "prefix. Call reset() and prefill again.")
        self.reset()

    def __repr__(self) -> str:
        return (f"Qwen3_5Cache(full_layers={len(self.full_layers)}, linear_layers={len(self.linear_layers)}, "
                f"batch_size={self.batch_size}, max_seq_len={self.max_seq_len}, position={self.position})")


__all__ = ["Qwen3_5Cache"]
