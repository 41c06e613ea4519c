"""SigLIP vision-tower adapter (stand-alone use of the tower that Pi0.5 and other VLAs embed).

``SiglipAdapter(hf_vision_model).to_rpu()`` returns a callable ``model(pixel_values) -> last_hidden_state``.
Reference: ``python/rpu_backend/adapters/siglip.py`` (So400m/14 profile: 27 layers, width 1152, 16 heads of
72, MLP 4304), ``src/fused/rpu_siglip_model.cpp:1-40``.
"""
from __future__ import annotations

import torch

from ..models.vision import SiglipConfig, SiglipVisionEncoder
from ..runtime.errors import UnsupportedModelError


class SiglipAdapter:
    ARCHITECTURE = "SiglipVisionModel"

    @classmethod
    def preflight(cls, config) -> None:
        vc = getattr(config, "vision_config", config)
        if vc.hidden_size // vc.num_attention_heads > 256:
            raise UnsupportedModelError("SigLIP head size above 256 is not supported")
        if getattr(vc, "hidden_act", "gelu_pytorch_tanh") not in ("gelu_pytorch_tanh", "gelu"):
            raise UnsupportedModelError("SigLIP activation must be gelu_pytorch_tanh or gelu")

    def __init__(self, model, *, rpu_execution=None, dtype=torch.float16, prefix: str = "vision_model."):
        self.model, self.config = model, getattr(model.config, "vision_config", model.config)
        self.dtype, self.prefix, self._rpu_execution = dtype, prefix, rpu_execution
        self.preflight(self.config)

    def to_rpu(self, *, max_images: int = 8, projector=None, device="cuda") -> SiglipVisionEncoder:
        return SiglipVisionEncoder(SiglipConfig.from_hf(self.config), self.model.state_dict(), prefix=self.prefix,
                                   device=device, dtype=self.dtype, max_images=max_images, projector=projector)


__all__ = ["SiglipAdapter"]
