"""NVFP4 weights: 4-bit e2m1 codes, one e4m3 scale per 16 values along K, one fp32 scale per tensor.

Contract (the same as the reference's ``python/rpu_backend/quant/nvfp4_pack.py``):

* ``quantize_nvfp4(w[N,K]) -> (codes[N,K] uint8, scale_codes[K/16,N] uint8, tensor_scale fp32 scalar)``;
  the block scales are stored group-major with N contiguous;
* ``w ~ decode(code) * e4m3(scale_code[g,n]) * tensor_scale``;
* encoding saturates at +-6 and rounds to nearest with ties to the even code (0.25->0, 0.75->1.0, 1.25->1.0,
  1.75->2.0, 2.5->2.0, 3.5->4.0, 5.0->4.0); the sign bit comes from ``signbit`` so ``-0.0`` keeps it;
* ``tensor_scale = max(amax / (6 * 448), 2**-24)``.

``pack_nibbles`` / ``unpack_nibbles`` give the two-codes-per-byte form (even element in the low nibble) that the
device GEMM (``rf_gemm_w4``) streams.
"""
from __future__ import annotations

import torch

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
# halfway points between neighbouring magnitudes: value j sits between code j and code j + 1
_E2M1_MIDPOINTS = (E2M1_VALUES[:-1] + E2M1_VALUES[1:]) / 2
BLOCK = 16
_TENSOR_SCALE_FLOOR = 2.0 ** -24


def fp4_e2m1_encode(values: torch.Tensor) -> torch.Tensor:
    """fp32 -> e2m1 code (bit 3 sign, bits 0..2 magnitude index), saturating, round-to-nearest-even."""
    x = values.detach().to(torch.float32)
    mag = x.abs().clamp(max=6.0)
    mids = _E2M1_MIDPOINTS.to(x.device)
    below = torch.bucketize(mag, mids, right=False)      # a value ON a midpoint counts as below it
    above = torch.bucketize(mag, mids, right=True)       # ... or as above it
    # off a midpoint both agree; on one they differ by one and the even code wins
    idx = torch.where(below % 2 == 0, below, above)
    return idx.to(torch.uint8) | (torch.signbit(x).to(torch.uint8) << 3)


def fp4_e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    c = codes.to(torch.uint8)
    mag = E2M1_VALUES.to(c.device)[(c & 7).long()]
    return torch.where((c & 8) != 0, -mag, mag)


def quantize_nvfp4(weight: torch.Tensor):
    if weight.dim() != 2:
        raise ValueError(f"expected [N,K], got {tuple(weight.shape)}")
    N, K = weight.shape
    if K % BLOCK:
        raise ValueError(f"NVFP4 requires K divisible by {BLOCK}, got K={K}")
    w = weight.detach().float().reshape(N, K // BLOCK, BLOCK)
    tensor_scale = (w.abs().amax() / (6.0 * 448.0)).clamp_min(_TENSOR_SCALE_FLOOR).to(torch.float32)
    block_q = (w.abs().amax(-1) / (6.0 * tensor_scale)).clamp(0.0, 448.0).to(torch.float8_e4m3fn)
    eff = block_q.float() * tensor_scale                              # [N, K/16]
    dead = eff == 0                                                   # an all-zero block encodes as zeros
    unit = torch.where(dead, torch.ones_like(eff), eff)
    codes = fp4_e2m1_encode((w / unit[..., None]).clamp(-6.0, 6.0))
    codes = torch.where(dead[..., None], torch.zeros_like(codes), codes).reshape(N, K)
    return codes.contiguous(), block_q.view(torch.uint8).t().contiguous(), tensor_scale.contiguous()


def dequantize_nvfp4(codes: torch.Tensor, scale_codes_gn: torch.Tensor, tensor_scale: torch.Tensor) -> torch.Tensor:
    """The exact fp32 weight that ``(codes, scale_codes_gn, tensor_scale)`` stands for."""
    groups, N = scale_codes_gn.shape
    if tuple(codes.shape) != (N, groups * BLOCK):
        raise ValueError(f"codes {tuple(codes.shape)} incompatible with scales {tuple(scale_codes_gn.shape)}")
    eff = scale_codes_gn.t().contiguous().view(torch.float8_e4m3fn).float() * tensor_scale.float()
    return (fp4_e2m1_decode(codes).reshape(N, groups, BLOCK) * eff[..., None]).reshape(N, groups * BLOCK)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[N, K] 4-bit codes -> [N, K/2] bytes, element 2i in the low nibble."""
    c = codes.to(torch.uint8) & 0xF
    return (c[:, 0::2] | (c[:, 1::2] << 4)).contiguous()


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    return torch.stack((packed & 0xF, packed >> 4), -1).flatten(-2)


__all__ = ["quantize_nvfp4", "dequantize_nvfp4", "fp4_e2m1_encode", "fp4_e2m1_decode", "pack_nibbles",
           "unpack_nibbles", "E2M1_VALUES", "BLOCK"]
