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


__all__ = ["rope_tables", "mrope_axis_of_freq", "partial_rotary_dim", "baked_interleaved_tables"]
