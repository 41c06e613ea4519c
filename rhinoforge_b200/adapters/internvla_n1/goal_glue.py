"""Goal glue of InternVLA-N1: four language-model tokens become one goal token for the navigation head.

Two small fp32 modules that stay on the CPU (a few hundred kFLOP per call - moving them to the GPU would cost more in
launches than it saves):

* ``vlm_embed_mlp``: ``3584 -> 896 -> 448 -> 384`` with ReLU between the layers;
* ``goal_compressor``: one learned query attends over the four projected tokens (8 heads), with learned positional
  embeddings added to tokens and query.

Parameter names follow the checkpoint file ``navdp_head.safetensors`` (prefixes ``vlm_embed_mlp.`` and
``goal_compressor.``) so that it loads strictly.  Reference: ``python/rpu_backend/adapters/internvla_n1/goal_glue.py:1-96``.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Union

import torch
import torch.nn as nn

VLM_DIM, TOKEN_DIM, HEADS, MAX_POSITIONS = 3584, 384, 8, 5000
LEGACY_PE_KEY, LEGACY_PE_ROWS = "positional_encoding.pe", 1000


class _LearnedPositions(nn.Module):
    def __init__(self, dim: int, max_len: int = MAX_POSITIONS):
        super().__init__()
        self.position_embedding = nn.Embedding(max_len, dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.position_embedding.weight[:x.shape[1]].unsqueeze(0).expand(x.shape[0], -1, -1)


class TokenCompressor(nn.Module):
    """``[B, S, E] -> [B, target_length, E]``: learned queries cross-attend over the tokens."""

    def __init__(self, embed_dim: int = TOKEN_DIM, num_heads: int = HEADS, target_length: int = 1):
        super().__init__()
        self.target_embedding = nn.Embedding(target_length, embed_dim)
        self.token_positional_encoding = _LearnedPositions(embed_dim)
        self.query_positional_encoding = _LearnedPositions(embed_dim)
        self.cross_attention = nn.MultiheadAttention(embed_dim, num_heads, batch_first=True)
        self.embed_dim, self.num_heads = embed_dim, num_heads

    def forward(self, tokens: torch.Tensor, padding_mask: torch.Tensor = None) -> torch.Tensor:
        tokens = tokens + self.token_positional_encoding(tokens)
        query = self.target_embedding.weight.unsqueeze(0).expand(tokens.shape[0], -1, -1)
        query = query + self.query_positional_encoding(query)
        out, _ = self.cross_attention(query, tokens, tokens, key_padding_mask=padding_mask, need_weights=False)
        return out


class GoalGlue(nn.Module):
    def __init__(self, vlm_dim: int = VLM_DIM, token_dim: int = TOKEN_DIM):
        super().__init__()
        self.vlm_embed_mlp = nn.Sequential(nn.Linear(vlm_dim, vlm_dim // 4), nn.ReLU(),
                                           nn.Linear(vlm_dim // 4, vlm_dim // 8), nn.ReLU(),
                                           nn.Linear(vlm_dim // 8, token_dim))
        self.goal_compressor = TokenCompressor(token_dim, HEADS, 1)

    def forward(self, vlm_tokens: torch.Tensor) -> torch.Tensor:
        return self.goal_compressor(self.vlm_embed_mlp(vlm_tokens))


def load_goal_glue_state(glue: GoalGlue, tensors: Dict[str, torch.Tensor]) -> GoalGlue:
    """Strict load of the two prefixes from a flat tensor mapping.  Older files also carry an unused sinusoidal table
    ``goal_compressor.positional_encoding.pe`` of 1000 rows; it is dropped after its shape is checked."""
    part = lambda prefix: {k[len(prefix):]: v.float() for k, v in tensors.items() if k.startswith(prefix)}
    glue.vlm_embed_mlp.load_state_dict(part("vlm_embed_mlp."), strict=True)
    comp = part("goal_compressor.")
    legacy = comp.pop(LEGACY_PE_KEY, None)
    if legacy is not None and tuple(legacy.shape) != (LEGACY_PE_ROWS, glue.goal_compressor.embed_dim):
        raise ValueError(f"InternVLA-N1 legacy {LEGACY_PE_KEY} must have shape "
                         f"({LEGACY_PE_ROWS}, {glue.goal_compressor.embed_dim}), got {tuple(legacy.shape)}")
    glue.goal_compressor.load_state_dict(comp, strict=True)
    return glue


def build_goal_glue(safetensors_path: Union[str, Path], device: str = "cpu") -> GoalGlue:
    """The glue with the weights of ``navdp_head.safetensors``, fp32, in eval mode, on the CPU (the only placement)."""
    if device != "cpu":
        raise ValueError("InternVLA-N1 goal glue supports only device='cpu' with fp32")
    from safetensors.torch import load_file
    return load_goal_glue_state(GoalGlue().eval(), load_file(str(safetensors_path))).float().cpu()


__all__ = ["GoalGlue", "TokenCompressor", "build_goal_glue", "load_goal_glue_state"]
