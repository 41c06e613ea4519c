"""InternVLA-N1 RGB-D encoder builder: ``rgbd_encoder.*`` of ``navdp_head.safetensors`` ->
:class:`rhinoforge_b200.models.rgbd.RgbdEncoder` (``device="cuda"``) or its fp32 PyTorch statement (``device="cpu"``).

The DINOv2 towers are built from the tensors alone - no external DINOv2 source tree is imported.
Reference: ``python/rpu_backend/adapters/internvla_n1/rgbd.py:149-162`` (strict load of the ``rgbd_encoder.`` prefix).
"""
from __future__ import annotations

from pathlib import Path
from typing import Mapping, Optional, Union

import torch

from ...models.rgbd import RgbdConfig, RgbdEncoder, TorchRgbdEncoder, rgbd_shapes
from .._assets import verify_asset_manifest

PREFIX = "rgbd_encoder."


def rgbd_state_dict(tensors: Mapping[str, torch.Tensor], cfg: Optional[RgbdConfig] = None):
    cfg = cfg or RgbdConfig()
    local = {k[len(PREFIX):]: v for k, v in tensors.items() if k.startswith(PREFIX)}
    if not local:
        raise ValueError(f"no `{PREFIX}*` tensors in the checkpoint")
    want = {n for n, _, _ in rgbd_shapes(cfg)}
    ignored = {"rgb_model.mask_token", "depth_model.mask_token"}
    extra = sorted(set(local) - want - ignored)
    missing = sorted(want - set(local))
    if extra or missing:
        raise ValueError(f"RGB-D encoder tensors do not match the profile: missing {missing[:4]}, unexpected {extra[:4]}")
    return {k: v for k, v in local.items() if k in want}


def build_rgbd_encoder(safetensors_path: Union[str, Path], *, device: str = "cuda", dtype=torch.float16, max_batch: int = 1,
                       asset_manifest: Optional[Mapping] = None, config: Optional[RgbdConfig] = None):
    path = Path(safetensors_path).expanduser().resolve()
    verify_asset_manifest((path,), asset_manifest)
    from safetensors.torch import load_file
    cfg = config or RgbdConfig()
    sd = rgbd_state_dict(load_file(str(path)), cfg)
    if str(device).startswith("cpu"):
        return TorchRgbdEncoder(cfg, sd)
    return RgbdEncoder(cfg, sd, max_batch=max_batch, device=device, dtype=dtype)


__all__ = ["build_rgbd_encoder", "rgbd_state_dict", "PREFIX"]
