"""Group-wise int4: one fp16 scale per (output channel, K-block of 32/64/128).
Reference: ``python/rpu_backend/quant/int4_pgrp_pack.py``."""
from __future__ import annotations

import torch

from .int4_pack import pack_int4, unpack_int4

GROUP_SIZES = (32, 64, 128)


def quantize_pack_int4_pgrp(weight: torch.Tensor, group_size: int = 32):
    if group_size not in GROUP_SIZES:
        raise ValueError(f"group_size must be one of {GROUP_SIZES}, got {group_size}")
    N, K = weight.shape
    if K % group_size:
        raise ValueError(f"K={K} is not a multiple of the group size {group_size}")
    w = weight.detach().float().view(N, K // group_size, group_size)
    scale = (w.abs().amax(-1) / 7.0).to(torch.float16).clamp_min(torch.finfo(torch.float16).tiny)
    q = torch.round(w / scale.float()[..., None]).clamp_(-8, 7).to(torch.int8).view(N, K)
    return pack_int4(q), scale


def dequantize_int4_pgrp(packed: torch.Tensor, scale: torch.Tensor, group_size: int = 32) -> torch.Tensor:
    q = unpack_int4(packed).float()
    N, K = q.shape
    return (q.view(N, K // group_size, group_size) * scale.float()[..., None]).view(N, K).to(torch.float16)
