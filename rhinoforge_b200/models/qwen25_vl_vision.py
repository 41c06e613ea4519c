"""Qwen2.5-VL vision transformer on the native stack (the image tower of Wall-OSS).

32 RMSNorm blocks (hidden 1280, 16 heads of 80, SwiGLU MLP 3420 with biases on every projection), 2-D
rotate-half RoPE, *window attention*: all blocks but ``fullatt_block_indexes`` attend inside 112 x 112-pixel
windows (4 x 4 merged patches).  The reference builds a block-diagonal mask for those layers
(``src/fused/rpu_qwen25vl_vision_model.cpp:1-17``); here the tokens are reordered window by window once (as
the Hugging Face module does) and a window is simply one *sequence* of the varlen attention launch, so the
windowed blocks do no masked work at all.  The stack is driven in runs of consecutive blocks that share a
sequence partition (``layer_range``): windows, full image, windows, ...  The merger (RMSNorm over each patch,
``fc -> GELU -> fc`` over groups of ``merge^2`` patches) runs on the GEMM kernel and the rows go back to
raster order at the end.

Head size 80 runs on the 128-wide attention kernels with zero-padded heads; the intermediate size is padded
to a multiple of 64 with zero rows/columns (the reference pads 3420 to 3456 for the same reason).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch

from ..ops import kernels as K
from ..runtime.errors import RPUBackendError
from ..runtime.stack import pad_heads
from .vision import TowerGeometry, VisionTower, padded_head_dim, rope2d_tables


@dataclass
class Qwen25VLVisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    patch_size: int = 14
    temporal_patch_size: int = 2
    in_channels: int = 3
    spatial_merge_size: int = 2
    window_size: int = 112
    out_hidden_size: int = 3584
    fullatt_block_indexes: Tuple[int, ...] = (7, 15, 23, 31)
    hidden_act: str = "silu"

    @classmethod
    def from_hf(cls, c) -> "Qwen25VLVisionConfig":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        return cls(**{f: (tuple(g(f)) if f == "fullatt_block_indexes" else g(f))
                      for f in cls.__dataclass_fields__ if g(f) is not None})


def window_partition(grid: Sequence[Tuple[int, int, int]], merge: int, window_units: int):
    """Window order of the merged-patch units of a batch of images / videos.

    ``grid`` holds ``(t, h, w)`` in patches; a unit is a ``merge x merge`` patch group and a window is
    ``window_units x window_units`` units (ragged at the right and bottom edges).  Returns ``(order, lens)``:
    ``order[i]`` is the raster index of the unit that sits at position ``i`` of the window-major order, and
    ``lens`` the number of units of each (non-empty) window in that order.  Windows never span frames."""
    order: List[int] = []
    lens: List[int] = []
    base = 0
    for t, h, w in grid:
        uh, uw = h // merge, w // merge
        for f in range(t):
            for wy in range(0, uh, window_units):
                for wx in range(0, uw, window_units):
                    ys = range(wy, min(wy + window_units, uh))
                    xs = range(wx, min(wx + window_units, uw))
                    order += [base + f * uh * uw + y * uw + x for y in ys for x in xs]
                    lens.append(len(ys) * len(xs))
        base += t * uh * uw
    return order, lens


def _pad_rows(w: torch.Tensor, rows: int) -> torch.Tensor:
    if w.shape[0] == rows:
        return w
    out = w.new_zeros((rows,) + tuple(w.shape[1:]))
    out[:w.shape[0]] = w
    return out


class Qwen25VLVisionEncoder:
    """``forward(pixel_values, grid_thw)`` -> image embeddings ``[T / merge^2, out_hidden]`` in raster order.

    ``pixel_values`` is the processor's flattened patch matrix ``[T, C*Tp*P*P]`` (merge-block order)."""

    def __init__(self, cfg: Qwen25VLVisionConfig, sd: Dict[str, torch.Tensor], *, prefix: str = "", device="cuda",
                 dtype=torch.float16, max_patches: int = 4096, max_windows: int = 1024):
        if cfg.hidden_act != "silu":
            raise RPUBackendError(f"unsupported Qwen2.5-VL vision activation {cfg.hidden_act}")
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        H, heads = cfg.hidden_size, cfg.num_heads
        hd = H // heads
        hd_pad = padded_head_dim(hd)
        inter = (cfg.intermediate_size + 63) // 64 * 64
        g = lambda n: sd[prefix + n]
        pw = g("patch_embed.proj.weight").reshape(H, -1)
        self.k_patch = pw.shape[1]
        k_pad = (self.k_patch + 7) // 8 * 8
        self.patch_w = torch.nn.functional.pad(pw, (0, k_pad - self.k_patch)).to(self.device, dtype).contiguous()
        layers = []
        for i in range(cfg.depth):
            b = f"blocks.{i}."
            wqkv, bqkv = g(b + "attn.qkv.weight"), g(b + "attn.qkv.bias")
            wq, wk, wv = wqkv.view(3, heads * hd, H)
            bq, bk, bv = bqkv.view(3, heads * hd)
            wqkv_p = torch.cat([pad_heads(x, heads, hd, hd_pad, 0) for x in (wq, wk, wv)], 0)
            bqkv_p = torch.cat([pad_heads(x, heads, hd, hd_pad, 0) for x in (bq, bk, bv)], 0)
            w_up = torch.cat((_pad_rows(g(b + "mlp.gate_proj.weight"), inter), _pad_rows(g(b + "mlp.up_proj.weight"), inter)), 0)
            b_up = torch.cat((_pad_rows(g(b + "mlp.gate_proj.bias"), inter), _pad_rows(g(b + "mlp.up_proj.bias"), inter)), 0)
            w_down = torch.nn.functional.pad(g(b + "mlp.down_proj.weight"), (0, inter - cfg.intermediate_size))
            layers.append(dict(norm1_w=g(b + "norm1.weight"), wqkv=wqkv_p, bqkv=bqkv_p,
                               wo=pad_heads(g(b + "attn.proj.weight"), heads, hd, hd_pad, 1), bo=g(b + "attn.proj.bias"),
                               norm2_w=g(b + "norm2.weight"), w_up=w_up, b_up=b_up, w_down=w_down,
                               b_down=g(b + "mlp.down_proj.bias")))
        geo = TowerGeometry(H, cfg.depth, heads, hd, inter, 1e-6, "swiglu", "rms")
        self.tower = VisionTower(geo, layers, max_tokens=max_patches, max_seqs=max_windows, rotary=True,
                                 device=device, dtype=dtype)
        self.unit = cfg.spatial_merge_size ** 2
        t = lambda n: g(n).to(self.device, dtype).contiguous()
        self.ln_q = t("merger.ln_q.weight")
        self.m_w1, self.m_b1 = t("merger.mlp.0.weight"), t("merger.mlp.0.bias")
        self.m_w2, self.m_b2 = t("merger.mlp.2.weight"), t("merger.mlp.2.bias")
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))
        self.window_units = max(1, cfg.window_size // cfg.spatial_merge_size // cfg.patch_size)
        full = set(int(i) for i in cfg.fullatt_block_indexes)
        # runs of consecutive blocks that share one sequence partition: (first, last + 1, full attention?)
        self.segments: List[Tuple[int, int, bool]] = []
        for i in range(cfg.depth):
            f = i in full
            if self.segments and self.segments[-1][2] == f:
                self.segments[-1] = (self.segments[-1][0], i + 1, f)
            else:
                self.segments.append((i, i + 1, f))
        self._geom_cache: Dict[tuple, tuple] = {}

    def _geometry(self, grid: Tuple[Tuple[int, int, int], ...]):
        hit = self._geom_cache.get(grid)
        if hit is not None:
            return hit
        m, dev = self.cfg.spatial_merge_size, self.device
        max_hw = max(max(h, w) for _, h, w in grid)
        cos, sin, axis, _ = rope2d_tables(range(max_hw), range(max_hw), self.inv_freq)
        pos_parts, frame_lens = [], []
        for t, h, w in grid:
            r = torch.arange(h).view(h // m, 1, m, 1).expand(h // m, w // m, m, m).reshape(-1)
            c = torch.arange(w).view(1, w // m, 1, m).expand(h // m, w // m, m, m).reshape(-1)
            pos_parts.append(torch.stack((r, max_hw + c), -1).repeat(t, 1))
            frame_lens += [h * w] * t
        order, win_units = window_partition(grid, m, self.window_units)
        order_t = torch.tensor(order, dtype=torch.long)
        pos = torch.cat(pos_parts).view(-1, self.unit, 2)[order_t].reshape(-1, 2)
        # full-attention sequences are whole frames; in window order a frame's units stay contiguous
        meta = {}
        for name, lens in (("win", [u * self.unit for u in win_units]), ("full", frame_lens)):
            l = torch.tensor(lens, dtype=torch.int32)
            meta[name] = ((torch.cumsum(l, 0, dtype=torch.int32) - l).to(dev), l.to(dev), int(l.max()))
        out = (order_t.to(dev), torch.argsort(order_t).to(dev), pos.to(dev, torch.int32).contiguous(), meta,
               cos.to(dev), sin.to(dev), axis.to(dev))
        self._geom_cache[grid] = out
        return out

    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        grid = tuple(tuple(int(v) for v in row) for row in (grid_thw.tolist() if torch.is_tensor(grid_thw) else grid_thw))
        order, inverse, pos, meta, cos, sin, axis = self._geometry(grid)
        T = pos.shape[0]
        if T > self.tower.max_tokens or meta["win"][0].numel() > self.tower.max_seqs:
            raise RPUBackendError(f"Qwen2.5-VL vision: {T} patches / {meta['win'][0].numel()} windows exceed the planned "
                                  f"{self.tower.max_tokens} / {self.tower.max_seqs}")
        x = pixel_values.to(self.device, self.dtype).reshape(T, -1)
        x = x.view(T // self.unit, self.unit, -1)[order].reshape(T, -1)          # window-major patch order
        if self.patch_w.shape[1] != x.shape[1]:
            x = torch.nn.functional.pad(x, (0, self.patch_w.shape[1] - x.shape[1]))
        hidden = K.gemm(x.contiguous(), self.patch_w)
        for first, last, is_full in self.segments:
            q_start, q_len, longest = meta["full" if is_full else "win"]
            self.tower.stack.forward(hidden, q_start=q_start, q_len=q_len, kv_len=q_len, max_q_len=longest,
                                     max_kv_len=longest, pos=pos, cos=cos, sin=sin, axis_of_freq=axis,
                                     layer_range=(first, last))
        y = K.rmsnorm(hidden, self.ln_q, 1e-6).view(T // self.unit, -1)
        y = K.gemm(K.gemm(y, self.m_w1, bias=self.m_b1, act="gelu_erf"), self.m_w2, bias=self.m_b2)
        return y[inverse]

    __call__ = forward

    def close(self):
        self.tower.close()


__all__ = ["Qwen25VLVisionConfig", "Qwen25VLVisionEncoder", "window_partition"]
