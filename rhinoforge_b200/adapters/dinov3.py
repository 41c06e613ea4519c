"""DINOv3 adapter: ``DINOv3Adapter.preflight(cfg); model = DINOv3Adapter(hf_model).to_rpu(); out = model(pixel_values)``.

Admitted by default: ViT-B/16 with 4 register tokens (hidden 768, 12 heads, 12 layers, patch 16).
Other plain-MLP geometries whose head size the attention kernels take (<= 256) can be admitted with
``RPU_DINOV3_ALLOW_ANY_PROFILE=1``; gated-MLP variants are always rejected.  The 12 heads are split
natively over tensor-parallel ranks (no padding to 16 heads as on 8-core parts).
Reference: ``python/rpu_backend/adapters/dinov3.py:77-142`` (profile gate), ``:159-342`` (install),
``:652-872`` (forward, RoPE tables), ``:937`` (adapter class).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..models.vision import DINOv3Config, DINOv3Encoder
from ..runtime.errors import RPUBackendError, UnsupportedModelError

PROFILE = dict(hidden_size=768, num_attention_heads=12, num_hidden_layers=12, patch_size=16, num_register_tokens=4)


class _DINOv3Handle:
    """Callable runtime handle; returns ``BaseModelOutputWithPooling(last_hidden_state, pooler_output=CLS)``."""

    def __init__(self, encoder: DINOv3Encoder, config, execution=None):
        self.encoder, self.config, self._rpu_execution = encoder, config, execution
        self._rpu_is_ready = True

    @property
    def device(self):
        return self.encoder.device

    @property
    def dtype(self):
        return self.encoder.dtype

    def eval(self):
        return self

    def to(self, device=None, *a, **kw):
        name = str(device).lower() if device is not None else ""
        if device is None or name.startswith(("rpu", "cuda")):
            return self
        raise RPUBackendError("this model's weights were packed for the accelerator exactly once; reload the checkpoint")

    @torch.no_grad()
    def forward(self, pixel_values: torch.Tensor, return_dict: bool = True, **kw):
        last, pooled = self.encoder(pixel_values)
        self.encoder.tower.stack.check_status()
        if not return_dict:
            return last, pooled
        from transformers.modeling_outputs import BaseModelOutputWithPooling
        return BaseModelOutputWithPooling(last_hidden_state=last, pooler_output=pooled)

    __call__ = forward

    def close(self):
        self.encoder.close()


class DINOv3Adapter:
    ARCHITECTURE = "DINOv3ViTModel"
    EXECUTION_STAGES = {"vision": ("chunk_size",)}

    @classmethod
    def preflight(cls, config) -> None:
        g = lambda k, d=None: getattr(config, k, d)
        if g("use_gated_mlp", False):
            raise UnsupportedModelError("DINOv3 gated-MLP variants are not supported")
        if os.environ.get("RPU_DINOV3_ALLOW_ANY_PROFILE", "0") == "1":
            if g("hidden_size") // g("num_attention_heads") > 256:
                raise UnsupportedModelError("DINOv3 head size above 256 is not supported")
            return
        bad = {k: g(k) for k, v in PROFILE.items() if g(k) != v}
        if bad:
            raise UnsupportedModelError(f"DINOv3 profile not admitted (ViT-B/16 with 4 registers only): {bad}")

    @classmethod
    def preflight_execution(cls, config, execution) -> None:
        for stage in (execution or {}):
            if stage not in cls.EXECUTION_STAGES:
                raise UnsupportedModelError(f"DINOv3 has no execution stage {stage!r}")

    def __init__(self, model, *, rpu_execution=None, dtype=torch.float16):
        self.model, self.config = model, model.config
        self._rpu_execution, self.dtype = rpu_execution, dtype
        self.preflight(self.config)
        self.preflight_execution(self.config, rpu_execution)

    def to_rpu(self, *, max_images: int = 8, max_patches_per_image: Optional[int] = None, device="cuda"):
        sd = self.model.state_dict()
        enc = DINOv3Encoder(DINOv3Config.from_hf(self.config), sd, device=device, dtype=self.dtype,
                            max_images=max_images, max_patches_per_image=max_patches_per_image)
        return _DINOv3Handle(enc, self.config, self._rpu_execution)


__all__ = ["DINOv3Adapter"]
