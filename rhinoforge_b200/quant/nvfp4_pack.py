"""NVFP4-style weights: e2m1 codes, one unsigned 8-bit (e4m3-coded) scale per 16 values, one fp32
scale per tensor.  Reference: ``python/rpu_backend/quant/nvfp4_pack.py``."""
from __future__ import annotations

import torch

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
BLOCK = 16


def _to_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code (bit 3 = sign, bits 0..2 = magnitude index)."""
    mag = x.abs()[..., None]
    idx = (mag - E2M1_VALUES.to(x.device)).abs().argmin(-1).to(torch.uint8)
    return idx | ((x < 0).to(torch.uint8) << 3)


def quantize_nvfp4(weight: torch.Tensor):
    N, K = weight.shape
    if K % BLOCK:
        raise ValueError(f"K={K} is not a multiple of {BLOCK}")
    w = weight.detach().float().view(N, K // BLOCK, BLOCK)
    tensor_scale = (w.abs().amax() / (6.0 * 448.0)).clamp_min(1e-12)
    block = (w.abs().amax(-1) / 6.0 / tensor_scale).clamp(0, 448.0)
    block_q = block.to(torch.float8_e4m3fn)
    eff = block_q.float() * tensor_scale
    codes = _to_e2m1(w / eff.clamp_min(1e-30)[..., None]).view(N, K)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return packed, block_q.view(torch.uint8), tensor_scale.to(torch.float32)


def dequantize_nvfp4(packed: torch.Tensor, block_scale_u8: torch.Tensor, tensor_scale: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    codes = torch.stack((lo, hi), -1).flatten(-2)
    vals = E2M1_VALUES.to(packed.device)[(codes & 7).long()] * torch.where((codes & 8) > 0, -1.0, 1.0)
    N, K = vals.shape
    s = block_scale_u8.view(torch.float8_e4m3fn).float() * tensor_scale
    return (vals.view(N, K // BLOCK, BLOCK) * s[..., None]).view(N, K).to(torch.float16)
