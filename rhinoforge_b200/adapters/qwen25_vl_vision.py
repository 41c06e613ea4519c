"""Qwen2.5-VL vision-tower adapter (the image tower of Wall-OSS, usable on its own).

``Qwen25VLVisionAdapter(hf_visual).to_rpu()`` returns a callable ``model(pixel_values, grid_thw) -> image_embeds``
(``[patches / merge^2, out_hidden]`` in raster order).  Reference: ``python/rpu_backend/adapters/wall_oss/vision.py``
(32 blocks, hidden 1280, 16 heads of 80, SwiGLU 3420 with biases, window attention with full-attention blocks
7/15/23/31), ``src/fused/rpu_qwen25vl_vision_model.cpp:1-17``.
"""
from __future__ import annotations

import torch

from ..models.qwen25_vl_vision import Qwen25VLVisionConfig, Qwen25VLVisionEncoder
from ..runtime.errors import UnsupportedModelError


class Qwen25VLVisionAdapter:
    ARCHITECTURE = "Qwen2_5_VisionTransformerPretrainedModel"

    @classmethod
    def preflight(cls, config) -> None:
        vc = getattr(config, "vision_config", config)
        g = (lambda k, d=None: vc.get(k, d)) if isinstance(vc, dict) else (lambda k, d=None: getattr(vc, k, d))
        if g("hidden_act", "silu") != "silu":
            raise UnsupportedModelError("Qwen2.5-VL vision activation must be silu")
        hd = g("hidden_size") // g("num_heads")
        if hd > 256 or hd % 4:
            raise UnsupportedModelError(f"Qwen2.5-VL vision head size {hd} is not supported (<= 256, multiple of 4)")
        unit = g("spatial_merge_size", 2) * g("patch_size", 14)
        if g("window_size", 112) % unit:
            raise UnsupportedModelError("window_size must be a multiple of spatial_merge_size * patch_size")
        full = list(g("fullatt_block_indexes", ()))
        if any(i < 0 or i >= g("depth") for i in full):
            raise UnsupportedModelError("fullatt_block_indexes out of range")

    def __init__(self, model, *, rpu_execution=None, dtype=torch.float16, prefix: str = ""):
        self.model, self.config = model, getattr(model.config, "vision_config", model.config)
        self.dtype, self.prefix, self._rpu_execution = dtype, prefix, rpu_execution
        self.preflight(self.config)

    def to_rpu(self, *, max_patches: int = 4096, max_windows: int = 1024, device="cuda") -> Qwen25VLVisionEncoder:
        return Qwen25VLVisionEncoder(Qwen25VLVisionConfig.from_hf(self.config), self.model.state_dict(), prefix=self.prefix,
                                     device=device, dtype=self.dtype, max_patches=max_patches, max_windows=max_windows)


__all__ = ["Qwen25VLVisionAdapter"]
