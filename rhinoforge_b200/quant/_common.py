"""Per-output-channel symmetric weight quantisation shared by the converters and the loader.

``W ~= scale[:, None] * Q`` with ``Q`` int8 in [-127, 127] (or [-8, 7] stored in int8 containers
for 4-bit probes) and one fp16 scale per output row.  The runtime computes ``(X . Q^T) * scale``
in fp32, the order this module's ``reference_linear`` uses.  Semantics of the reference:
``python/rpu_backend/quant/_common.py:10-41``.
"""
from __future__ import annotations

from typing import Tuple

import torch

_FP16_TINY = torch.finfo(torch.float16).tiny


def quantize_linear_per_channel(weight: torch.Tensor, *, bits: int = 8) -> Tuple[torch.Tensor, torch.Tensor]:
    if weight.dim() != 2:
        raise ValueError(f"expected 2-D Linear weight, got {tuple(weight.shape)}")
    if bits not in (4, 8):
        raise ValueError(f"expected bits to be 4 or 8, got {bits}")
    qmax, qmin = (1 << (bits - 1)) - 1, -(1 << (bits - 1))
    w = weight.detach().to(torch.float16).to(torch.float32)
    scale = (w.abs().amax(dim=1) / float(qmax)).to(torch.float16).clamp_min(_FP16_TINY)
    q = torch.round(w / scale.to(torch.float32)[:, None]).clamp_(qmin, qmax).to(torch.int8)
    return q, scale


def dequantize_linear_per_channel(w_int8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return scale.to(torch.float16)[:, None] * w_int8.to(torch.float16)


def reference_linear(x: torch.Tensor, w_int8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 oracle of the W8A16 kernels: accumulate ``x . q^T`` exactly, scale once per channel."""
    return (x.float() @ w_int8.float().t()) * scale.float()


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.flatten().float(), b.flatten().float()
    return float(torch.dot(a, b) / (a.norm() * b.norm()).clamp_min(1e-30))


__all__ = ["quantize_linear_per_channel", "dequantize_linear_per_channel", "reference_linear", "cosine"]
