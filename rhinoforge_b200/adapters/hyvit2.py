"""HYViT2 vision-tower adapter (the HunYuan embodied VLA's image tower, usable on its own).

``HYViT2Adapter(config, state_dict).to_rpu(projector=(w, b))`` returns a callable ``model(pixel_values) -> features``:
the SigLIP-So400m body without the post-LayerNorm, timm-style checkpoint names, an optional per-token projector (the
first linear of the merger).  Reference: ``src/fused/rpu_hyvit2_vision_model.cpp:1-30``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..models.vision import HYViT2Encoder, SiglipConfig
from ..runtime.errors import UnsupportedModelError


class HYViT2Adapter:
    ARCHITECTURE = "HYViT2VisionTransformer"

    @classmethod
    def preflight(cls, config) -> None:
        c = SiglipConfig.from_hf(config)
        if c.hidden_size % c.num_attention_heads or c.hidden_size // c.num_attention_heads > 256:
            raise UnsupportedModelError("HYViT2 head size must divide the width and be at most 256")
        if c.image_size % c.patch_size:
            raise UnsupportedModelError("HYViT2 image size must be a multiple of the patch size")
        if c.hidden_act not in ("gelu_pytorch_tanh", "gelu"):
            raise UnsupportedModelError("HYViT2 activation must be gelu_pytorch_tanh or gelu")

    def __init__(self, config, state_dict: Dict[str, torch.Tensor], *, rpu_execution=None, dtype=torch.float16,
                 prefix: str = ""):
        self.config, self.sd, self.dtype, self.prefix, self._rpu_execution = config, state_dict, dtype, prefix, rpu_execution
        self.preflight(config)

    def to_rpu(self, *, max_images: int = 1, projector: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
               device="cuda") -> HYViT2Encoder:
        return HYViT2Encoder(SiglipConfig.from_hf(self.config), self.sd, prefix=self.prefix, device=device,
                             dtype=self.dtype, max_images=max_images, projector=projector)


__all__ = ["HYViT2Adapter"]
