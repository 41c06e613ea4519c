"""Packed int4 weights with one fp16 scale per output channel (two nibbles per byte, low first).
Reference layout: ``python/rpu_backend/quant/int4_pack.py``."""
from __future__ import annotations

import torch

from ._common import quantize_linear_per_channel


def pack_int4(q: torch.Tensor) -> torch.Tensor:
    """[N, K] int8 values in [-8, 7] -> [N, K/2] uint8 (element 2i in the low nibble)."""
    if q.shape[-1] % 2:
        raise ValueError("K must be even to pack two int4 values per byte")
    u = (q.to(torch.int16) & 0xF).to(torch.uint8)
    return u[..., 0::2] | (u[..., 1::2] << 4)


def unpack_int4(p: torch.Tensor) -> torch.Tensor:
    lo = (p & 0xF).to(torch.int8)
    hi = (p >> 4).to(torch.int8)
    lo = torch.where(lo > 7, lo - 16, lo)
    hi = torch.where(hi > 7, hi - 16, hi)
    return torch.stack((lo, hi), -1).flatten(-2)


def quantize_pack_int4(weight: torch.Tensor):
    q, scale = quantize_linear_per_channel(weight, bits=4)
    return pack_int4(q), scale
