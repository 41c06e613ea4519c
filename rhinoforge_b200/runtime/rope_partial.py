"""Host builders of rotary tables: 1-D, sectioned / interleaved M-RoPE, partial rotary and 2-D vision RoPE
(reference: ``python/rpu_backend/runtime/rope_partial.py:129,176``).  The kernels take fp32 ``cos``/``sin`` tables
``[positions, rot_dim/2]`` plus an optional per-frequency axis selector; these helpers produce both."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch


def rope_tables(rot_dim: int, max_pos: int, theta: float = 10000.0, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None]
    return ang.cos().contiguous(), ang.sin().contiguous()


def mrope_axis_of_freq(rot_dim: int, section: Sequence[int], interleaved: bool = True) -> torch.Tensor:
    """Axis (0 = T, 1 = H, 2 = W) of every rotary frequency: interleaved ``THWTHW...TT`` or chunked ``T..H..W..``."""
    half = rot_dim // 2
    if sum(section) != half:
        raise ValueError(f"mrope_section {tuple(section)} must sum to rot_dim/2 = {half}")
    axis = torch.zeros(half, dtype=torch.int8)
    if interleaved:
        for dim, off in ((1, 1), (2, 2)):
            axis[off:section[dim] * 3:3] = dim
    else:
        axis[section[0]:section[0] + section[1]] = 1
        axis[section[0] + section[1]:] = 2
    return axis


def partial_rotary_dim(head_dim: int, factor: float) -> int:
    rot = int(head_dim * factor)
    if rot <= 0 or rot % 2 or rot > head_dim:
        raise ValueError(f"partial rotary factor {factor} gives an invalid rotary width {rot} for head_dim {head_dim}")
    return rot


def baked_interleaved_tables(positions3: torch.Tensor, rot_dim: int, section: Sequence[int], theta: float = 10000.0,
                             interleaved: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token cos/sin ``[tokens, rot_dim/2]`` with the axis choice already applied (``positions3`` is ``[3, tokens]``):
    what a kernel without an axis selector would be fed."""
    axis = mrope_axis_of_freq(rot_dim, section, interleaved).long()
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    pos = positions3.float()[axis, :].t()                      # [tokens, half]
    ang = pos * inv[None]
    return ang.cos().contiguous(), ang.sin().contiguous()


def _mrope_tables(position_ids: torch.Tensor, head_dim: int, rope_theta: float, mrope_section: Sequence[int],
                  rotary_dim, interleaved: bool, builder: str) -> Tuple[torch.Tensor, torch.Tensor]:
    if not isinstance(position_ids, torch.Tensor) or position_ids.dim() != 2 or position_ids.shape[1] != 3:
        raise ValueError(f"{builder}: position_ids must be [seq, 3] (T/H/W coordinates), got "
                         f"{tuple(getattr(position_ids, 'shape', ()))}")
    if position_ids.is_floating_point() or position_ids.dtype == torch.bool:
        raise TypeError(f"{builder}: position_ids must be an integer tensor, got {position_ids.dtype}")
    if position_ids.numel() and int(position_ids.min()) < 0:
        raise ValueError(f"{builder}: position_ids must be non-negative, got minimum {int(position_ids.min())}")
    rot = head_dim if rotary_dim is None else int(rotary_dim)
    if rot <= 0 or rot % 2 or rot > head_dim:
        raise ValueError(f"{builder}: rotary_dim {rot} must be even and within head_dim {head_dim}")
    if not rope_theta > 0:
        raise ValueError(f"{builder}: rope_theta must be positive, got {rope_theta}")
    section = [int(v) for v in mrope_section]
    if len(section) != 3 or min(section) < 0 or sum(section) != rot // 2:
        raise ValueError(f"{builder}: mrope_section {section} must be three non-negative pair counts summing to "
                         f"rotary_dim/2 = {rot // 2}")
    axis = mrope_axis_of_freq(rot, section, interleaved).long()
    inv = 1.0 / (float(rope_theta) ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))
    ang = position_ids.to("cpu", torch.float64)[:, axis] * inv[None]                 # [seq, rot/2]
    cos, sin = ang.cos().to(torch.float16).contiguous(), ang.sin().to(torch.float16).contiguous()
    if not (torch.isfinite(cos).all() and torch.isfinite(sin).all()):
        raise ValueError(f"{builder}: non-finite table entries")
    return cos, sin


def build_interleaved_mrope_cos_sin(position_ids: torch.Tensor, *, head_dim: int, rope_theta: float,
                                    mrope_section: Sequence[int], rotary_dim=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Qwen3-VL tables, fp16 ``[seq, rotary_dim/2]`` on the CPU, for ``position_ids [seq, 3]``: T is the baseline of
    every frequency, H takes frequencies ``1 + 3i`` and W ``2 + 3i`` (as many as their section holds)."""
    return _mrope_tables(position_ids, head_dim, rope_theta, mrope_section, rotary_dim, True,
                         "build_interleaved_mrope_cos_sin")


def build_chunked_mrope_cos_sin(position_ids: torch.Tensor, *, head_dim: int, rope_theta: float,
                                mrope_section: Sequence[int], rotary_dim=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Qwen2.5-VL tables: contiguous frequency ranges ``[T x section[0], H x section[1], W x section[2]]``."""
    return _mrope_tables(position_ids, head_dim, rope_theta, mrope_section, rotary_dim, False,
                         "build_chunked_mrope_cos_sin")


__all__ = ["rope_tables", "mrope_axis_of_freq", "partial_rotary_dim", "baked_interleaved_tables",
           "build_interleaved_mrope_cos_sin", "build_chunked_mrope_cos_sin"]
