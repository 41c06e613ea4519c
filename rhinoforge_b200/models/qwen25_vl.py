"""Qwen2.5-VL: windowed-attention vision tower + Qwen2.5 text decoder (QKV bias, no QK norm) under chunked M-RoPE.

The text decoder is the generic :class:`rhinoforge_b200.runtime.engine.DecoderEngine`; what makes it Qwen2.5-VL is the
configuration (``attention_bias``, ``mrope_section`` with *contiguous* frequency ranges per axis: the first 16 rotary
pairs follow the temporal position, the next 24 the row and the last 24 the column) and the multimodal prefill: text
rows from the embedding kernel, merged image embeddings scattered over the placeholder rows, three-axis positions from
:func:`rhinoforge_b200.models.qwen3_vl.rope_index` (for still images Qwen2.5-VL and Qwen3-VL number positions the
same way).  There is no DeepStack.

Reference behaviour: ``python/rpu_backend/adapters/wall_oss/llm.py:1-30`` (Qwen2.5 = Qwen3 minus QK norm plus QKV
bias), ``adapters/wall_oss/vision.py:1-60`` (tower), ``runtime/rope_partial.py:129-176`` (chunked M-RoPE tables).
"""
from __future__ import annotations

from typing import Callable, Mapping, Optional

import torch

from ..ops import kernels as K
from ..runtime.engine import DecoderEngine
from ..runtime.errors import RPUBackendError, UnsupportedModelError
from .decoder import DecoderConfig
from .qwen25_vl_vision import Qwen25VLVisionConfig, Qwen25VLVisionEncoder
from .qwen3_vl import rope_index


def _cfg_get(c, k, d=None):
    return c.get(k, d) if isinstance(c, Mapping) else getattr(c, k, d)


def qwen25_text_config(hf_config) -> DecoderConfig:
    """Decoder configuration of a Qwen2.5-VL ``config.json`` (flat, or with a ``text_config`` block)."""
    tc = _cfg_get(hf_config, "text_config", None) or hf_config
    cfg = DecoderConfig.from_hf(tc)
    if cfg.mrope_section is None:
        raise UnsupportedModelError("Qwen2.5-VL text config carries no rope_scaling.mrope_section")
    import dataclasses
    return dataclasses.replace(cfg, mrope_interleaved=False, attention_bias=True, qk_norm=False)


class Qwen25VLEngine:
    """Vision encoder + decoder engine.  ``text_get(name)`` serves the decoder's tensors under the plain causal-LM names
    (``model.embed_tokens.weight``, ``model.layers.N.self_attn.q_proj.weight``, ..., ``model.norm.weight``,
    ``lm_head.weight``) and ``vision_sd[name]`` the tower's under ``blocks.N.*`` / ``merger.*`` / ``patch_embed.*``."""

    def __init__(self, cfg: DecoderConfig, vcfg: Qwen25VLVisionConfig, text_get: Callable[[str], torch.Tensor], vision_sd, *,
                 image_token_id: int = 151655, device="cuda", dtype=torch.float16, max_seq_len: int = 4096,
                 max_patches: int = 4096, max_prefill_tokens: int = 4096):
        if cfg.mrope_section is None or cfg.mrope_interleaved:
            raise UnsupportedModelError("Qwen2.5-VL needs chunked M-RoPE (mrope_section with mrope_interleaved=False)")
        self.cfg, self.vcfg, self.image_token_id = cfg, vcfg, image_token_id
        self.device, self.dtype = torch.device(device), dtype
        self.text = DecoderEngine(cfg, text_get, device=device, dtype=dtype, max_batch=1, max_seq_len=max_seq_len,
                                  max_prefill_tokens=max_prefill_tokens)
        self.vision = Qwen25VLVisionEncoder(vcfg, vision_sd, device=device, dtype=dtype, max_patches=max_patches)
        self._next_pos = 0

    @torch.no_grad()
    def prepare(self, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor] = None, image_grid_thw=None):
        """``(inputs_embeds [L, H], positions3 [3, L])`` of one sequence."""
        ids = input_ids.flatten().to("cpu")
        is_vis = ids == self.image_token_id
        grids = [] if image_grid_thw is None else [tuple(int(v) for v in g) for g in torch.as_tensor(image_grid_thw).tolist()]
        pos3 = rope_index(is_vis.to(torch.int32).tolist(), grids, self.vcfg.spatial_merge_size)
        embeds = torch.empty((ids.numel(), self.cfg.hidden_size), dtype=self.dtype, device=self.device)
        K.embedding(self.text.embed, ids.to(self.device, torch.int32), out=embeds, scale=self.cfg.embed_scale,
                    row_scale=self.text.embed_scale_rows)
        if pixel_values is not None:
            img = self.vision(pixel_values, grids)
            rows = is_vis.nonzero().flatten()
            if rows.numel() != img.shape[0]:
                raise RPUBackendError(f"{rows.numel()} image placeholder tokens but {img.shape[0]} image embeddings")
            K.scatter_rows(embeds, img, rows.to(self.device, torch.int32))
        elif bool(is_vis.any()):
            raise RPUBackendError("input_ids contain image placeholders but no pixel_values were given")
        return embeds, pos3

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor] = None, image_grid_thw=None, *,
                return_logits: bool = False):
        """Start sequence 0 from empty with a (possibly multimodal) prompt; returns the greedy next token."""
        self.text.reset()
        ids = input_ids.flatten()
        embeds, pos3 = self.prepare(ids, pixel_values, image_grid_thw)
        self._next_pos = int(pos3.max()) + 1
        return self.text.extend([ids], return_logits=return_logits, inputs_embeds=[embeds], positions3=[pos3])

    def decode(self, n_steps: int, **kw) -> torch.Tensor:
        out = self.text.decode(n_steps, **kw)
        self._next_pos += n_steps
        return out

    @torch.no_grad()
    def generate(self, input_ids, pixel_values=None, image_grid_thw=None, max_new_tokens: int = 16) -> torch.Tensor:
        first = self.prefill(input_ids, pixel_values, image_grid_thw)
        if max_new_tokens <= 1:
            return first[:, None]
        rest = self.decode(max_new_tokens - 1)
        self.text.check_status()
        return torch.cat((first[:, None], rest), 1)

    def close(self) -> None:
        self.vision.close()
        self.text.close()


__all__ = ["Qwen25VLEngine", "qwen25_text_config"]
