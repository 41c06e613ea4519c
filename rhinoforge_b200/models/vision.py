"""Vision towers on the native transformer stack: Qwen3-VL ViT, SigLIP, HYViT2 and DINOv3.

All three are a pre-norm LayerNorm ViT with a plain (non-gated) GELU MLP; they differ in patch
embedding, position information (interpolated learned table + 2-D RoPE / learned table / 2-D
RoPE on patch tokens only), extra tokens (CLS + registers), LayerScale, and what is read out
(patch merger + DeepStack taps / post-LN + projector / final LN + CLS pool).  Each family maps
its checkpoint names onto the stack's generic per-layer weight set; the layer loop itself is
``csrc/models/stack.cu`` with ``paged_kv=0`` (attention reads K/V from the fused QKV buffer,
one varlen launch for all images/frames).

Reference behaviour: ``src/fused/rpu_qwen3vl_vision_model.cpp:1-88`` (24-block ViT, 2-D RoPE,
DeepStack taps, merger), ``src/fused/rpu_siglip_model.cpp:142-200,1001-1215`` (in-graph patch
embed, packed multi-image forward, post-LN + projector), ``src/fused/rpu_dinov3_vision_model.cpp:1-16``
and ``python/rpu_backend/adapters/dinov3.py:652-872`` (CLS + registers, patch-only RoPE, LayerScale).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import kernels as K
from ..runtime.errors import RPUBackendError
from ..runtime.stack import NativeStack, StackSpec, pad_heads


def padded_head_dim(hd: int) -> int:
    for c in (64, 128, 256):
        if hd <= c:
            return c
    raise RPUBackendError(f"head_dim {hd} is larger than the attention kernels support (256)")


def fuse_qkv(wq, wk, wv, bq, bk, bv, heads: int, hd: int, hd_pad: int):
    """Fused, head-padded QKV weight ``[3*heads*hd_pad, hidden]`` and bias (missing biases are zero)."""
    ws, bs = [], []
    for w, b in ((wq, bq), (wk, bk), (wv, bv)):
        ws.append(pad_heads(w, heads, hd, hd_pad, 0))
        b = torch.zeros(heads * hd, dtype=w.dtype, device=w.device) if b is None else b
        bs.append(pad_heads(b, heads, hd, hd_pad, 0))
    return torch.cat(ws, 0), torch.cat(bs, 0)


def rope2d_tables(rows: Sequence[float], cols: Sequence[float], inv_freq: torch.Tensor, *, scale: float = 1.0):
    """cos/sin tables for 2-D rotate-half RoPE driven by integer table rows.

    The rotary half of a head holds ``[row-axis freqs | col-axis freqs]``, each ``len(inv_freq)`` wide.
    Table row ``i < len(rows)`` carries the angles of row coordinate ``rows[i]``, row ``len(rows)+j``
    those of column coordinate ``cols[j]``, and the last row is the identity rotation (for CLS and
    register tokens).  Returns ``(cos, sin, axis_of_freq, identity_row)``; a token's position pair is
    ``(row_index, len(rows) + col_index)``."""
    coords = torch.tensor(list(rows) + list(cols) + [0.0], dtype=torch.float64)
    ang = (scale * coords[:, None] * inv_freq.double()[None, :]).float()       # [R+C+1, F]
    ang = torch.cat((ang, ang), dim=1)                                            # both axis lanes share the table
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    F = inv_freq.numel()
    axis = torch.cat((torch.zeros(F, dtype=torch.int8), torch.ones(F, dtype=torch.int8)))
    return cos, sin, axis, len(coords) - 1


@dataclass
class TowerGeometry:
    hidden: int
    layers: int
    heads: int
    head_dim: int
    inter: int
    eps: float = 1e-6
    mlp: str = "gelu_tanh"
    norm: str = "layernorm"


class VisionTower:
    """A bidirectional ViT body on the native stack: ``run`` takes packed tokens of several images
    (or frames) and their per-sequence lengths; attention never crosses a sequence boundary."""

    def __init__(self, geo: TowerGeometry, layer_weights: List[Dict[str, torch.Tensor]], *, max_tokens: int,
                 max_seqs: int = 64, rotary: bool = False, device="cuda", dtype=torch.float16):
        self.geo, self.device, self.dtype = geo, torch.device(device), dtype
        self.hd_pad = padded_head_dim(geo.head_dim)
        spec = StackSpec(layers=geo.layers, hidden=geo.hidden, heads=geo.heads, kv_heads=geo.heads,
                         head_dim=self.hd_pad, inter=geo.inter, norm=geo.norm, mlp=geo.mlp, eps=geo.eps,
                         rot_dim=(geo.head_dim if rotary else 0), paged_kv=False, causal=False,
                         true_head_dim=geo.head_dim, max_tokens=max_tokens, max_seqs=max_seqs)
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.stack = NativeStack(spec, layer_weights, device=device, dtype=dtype)
        self._meta: Dict[tuple, tuple] = {}

    def run(self, hidden: torch.Tensor, seq_lens: Sequence[int], *, pos: Optional[torch.Tensor] = None,
            cos=None, sin=None, axis_of_freq=None, taps: Optional[Dict[int, torch.Tensor]] = None) -> torch.Tensor:
        T = hidden.shape[0]
        if T > self.max_tokens or len(seq_lens) > self.max_seqs or sum(seq_lens) != T:
            raise RPUBackendError(f"vision tower: {T} tokens / {len(seq_lens)} sequences exceed the planned "
                                  f"{self.max_tokens} / {self.max_seqs} (or lengths do not add up)")
        # sequence metadata is cached per partition: a repeated geometry launches no copy (and can be graph-captured)
        key = tuple(int(v) for v in seq_lens)
        meta = self._meta.get(key)
        if meta is None:
            lens = torch.tensor(list(key), dtype=torch.int32)
            starts = torch.cumsum(lens, 0, dtype=torch.int32) - lens
            dev = self.device
            meta = (starts.to(dev), lens.to(dev), int(lens.max()), torch.zeros(T, dtype=torch.int32, device=dev))
            if len(self._meta) < 64:
                self._meta[key] = meta
        q_start, q_len, longest, zero_pos = meta
        self.stack.forward(hidden, q_start=q_start, q_len=q_len, kv_len=q_len, max_q_len=longest, max_kv_len=longest,
                           pos=zero_pos if pos is None else pos, cos=cos, sin=sin, axis_of_freq=axis_of_freq, taps=taps)
        return hidden

    def close(self):
        self.stack.close()


# ----------------------------------------------------------------------------- Qwen3-VL ViT
@dataclass
class Qwen3VLVisionConfig:
    hidden_size: int = 1024
    depth: int = 24
    num_heads: int = 16
    intermediate_size: int = 4096
    patch_size: int = 16
    temporal_patch_size: int = 2
    in_channels: int = 3
    spatial_merge_size: int = 2
    out_hidden_size: int = 2048
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: Tuple[int, ...] = (5, 11, 17)
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_hf(cls, c) -> "Qwen3VLVisionConfig":
        g = (lambda k, d=None: c.get(k, d)) if isinstance(c, dict) else (lambda k, d=None: getattr(c, k, d))
        kw = {f: (tuple(g(f)) if f == "deepstack_visual_indexes" else g(f))
              for f in cls.__dataclass_fields__ if g(f) is not None}
        if "qwen3_5" in str(g("model_type", "")) and "deepstack_visual_indexes" not in kw:
            kw["deepstack_visual_indexes"] = ()          # the Qwen3.5 tower is this ViT without DeepStack taps
        return cls(**kw)


class _Merger:
    """LayerNorm -> fc1 + GELU(erf) -> fc2 over groups of merge*merge neighbouring patches."""

    def __init__(self, sd, prefix: str, group_dim: int, postshuffle: bool, dev, dtype):
        t = lambda n: sd[prefix + n].to(dev, dtype).contiguous()
        self.nw, self.nb = t("norm.weight"), t("norm.bias")
        self.w1, self.b1, self.w2, self.b2 = t("linear_fc1.weight"), t("linear_fc1.bias"), t("linear_fc2.weight"), t("linear_fc2.bias")
        self.group_dim, self.postshuffle = group_dim, postshuffle

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.postshuffle:
            y = K.layernorm(x.view(-1, self.group_dim), self.nw, self.nb, 1e-6)
        else:
            y = K.layernorm(x, self.nw, self.nb, 1e-6).view(-1, self.group_dim)
        return K.gemm(K.gemm(y, self.w1, bias=self.b1, act="gelu_erf"), self.w2, bias=self.b2)


class Qwen3VLVisionEncoder:
    """``forward(pixel_values, grid_thw)`` -> ``(image_embeds [T/merge^2, out_hidden], [deepstack feature] * n)``.

    ``pixel_values`` is the processor's flattened patch matrix ``[T, C*Tp*P*P]`` already in merge-block
    order; the Conv3d patch embedding is the same matrix product with the kernel flattened, and the
    bilinearly interpolated position table rides in as the GEMM's residual operand."""

    def __init__(self, cfg: Qwen3VLVisionConfig, sd: Dict[str, torch.Tensor], *, prefix: str = "", device="cuda",
                 dtype=torch.float16, max_patches: int = 4096, max_frames: int = 64):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        H, hd = cfg.hidden_size, cfg.hidden_size // cfg.num_heads
        if cfg.hidden_act not in ("gelu_pytorch_tanh", "gelu"):
            raise RPUBackendError(f"unsupported vision activation {cfg.hidden_act}")
        g = lambda n: sd[prefix + n]
        self.patch_w = g("patch_embed.proj.weight").reshape(H, -1).to(self.device, dtype).contiguous()
        self.patch_b = g("patch_embed.proj.bias").to(self.device, dtype).contiguous()
        self.pos_table = g("pos_embed.weight").to(self.device, torch.float32)
        self.grid_side = int(cfg.num_position_embeddings ** 0.5)
        layers = []
        for i in range(cfg.depth):
            b = f"blocks.{i}."
            layers.append(dict(norm1_w=g(b + "norm1.weight"), norm1_b=g(b + "norm1.bias"), wqkv=g(b + "attn.qkv.weight"),
                               bqkv=g(b + "attn.qkv.bias"), wo=g(b + "attn.proj.weight"), bo=g(b + "attn.proj.bias"),
                               norm2_w=g(b + "norm2.weight"), norm2_b=g(b + "norm2.bias"),
                               w_up=g(b + "mlp.linear_fc1.weight"), b_up=g(b + "mlp.linear_fc1.bias"),
                               w_down=g(b + "mlp.linear_fc2.weight"), b_down=g(b + "mlp.linear_fc2.bias")))
        geo = TowerGeometry(H, cfg.depth, cfg.num_heads, hd, cfg.intermediate_size, 1e-6,
                            "gelu_tanh" if cfg.hidden_act == "gelu_pytorch_tanh" else "gelu_erf")
        self.tower = VisionTower(geo, layers, max_tokens=max_patches, max_seqs=max_frames, rotary=True,
                                 device=device, dtype=dtype)
        unit = cfg.spatial_merge_size ** 2
        self.merger = _Merger(sd, prefix + "merger.", H * unit, False, self.device, dtype)
        self.ds_mergers = [_Merger(sd, f"{prefix}deepstack_merger_list.{j}.", H * unit, True, self.device, dtype)
                           for j in range(len(cfg.deepstack_visual_indexes))]
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))
        self._geom_cache: Dict[tuple, tuple] = {}

    # -- per-grid geometry: (row, col) table rows, interpolated position embeddings, frame lengths
    def _geometry(self, grid: Tuple[Tuple[int, int, int], ...]):
        hit = self._geom_cache.get(grid)
        if hit is not None:
            return hit
        m, side = self.cfg.spatial_merge_size, self.grid_side
        max_hw = max(max(h, w) for _, h, w in grid)
        cos, sin, axis, _ = rope2d_tables(range(max_hw), range(max_hw), self.inv_freq)
        pos_parts, emb_parts, lens = [], [], []
        for t, h, w in grid:
            r = torch.arange(h).view(h // m, 1, m, 1).expand(h // m, w // m, m, m).reshape(-1)
            c = torch.arange(w).view(1, w // m, 1, m).expand(h // m, w // m, m, m).reshape(-1)
            pos_parts.append(torch.stack((r, max_hw + c), -1).repeat(t, 1))
            hi, wi = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
            hf, wf = hi.int(), wi.int()
            hc, wc = (hf + 1).clip(max=side - 1), (wf + 1).clip(max=side - 1)
            dh, dw = (hi - hf)[:, None], (wi - wf)[None, :]
            tab = self.pos_table
            look = lambda a, b: tab[(a[:, None] * side + b[None, :]).reshape(-1).long().to(tab.device)].view(h, w, -1)
            wgt = lambda x: x.to(tab.device)[..., None]
            e = (look(hf, wf) * wgt((1 - dh) * (1 - dw)) + look(hf, wc) * wgt((1 - dh) * dw)
                 + look(hc, wf) * wgt(dh * (1 - dw)) + look(hc, wc) * wgt(dh * dw))
            e = e.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            emb_parts.append(e.repeat(t, 1))
            lens += [h * w] * t
        dev = self.device
        out = (torch.cat(pos_parts).to(dev, torch.int32).contiguous(), torch.cat(emb_parts).to(dev, self.dtype).contiguous(),
               lens, cos.to(dev), sin.to(dev), axis.to(dev))
        self._geom_cache[grid] = out
        return out

    def forward(self, pixel_values: torch.Tensor, grid_thw) -> Tuple[torch.Tensor, List[torch.Tensor]]:
        grid = tuple(tuple(int(v) for v in row) for row in (grid_thw.tolist() if torch.is_tensor(grid_thw) else grid_thw))
        pos, pos_emb, lens, cos, sin, axis = self._geometry(grid)
        x = pixel_values.to(self.device, self.dtype).reshape(pos.shape[0], -1).contiguous()
        hidden = K.gemm(x, self.patch_w, bias=self.patch_b, residual=pos_emb)
        taps = {int(l): torch.empty_like(hidden) for l in self.cfg.deepstack_visual_indexes}
        self.tower.run(hidden, lens, pos=pos, cos=cos, sin=sin, axis_of_freq=axis, taps=taps)
        deep = [mg(taps[int(l)]) for l, mg in zip(self.cfg.deepstack_visual_indexes, self.ds_mergers)]
        return self.merger(hidden), deep

    __call__ = forward

    def close(self):
        self.tower.close()


# ----------------------------------------------------------------------------- shared patchify
def patchify(pixel_values: torch.Tensor, patch: int, k_pad: int) -> torch.Tensor:
    """``[B, C, H, W]`` -> ``[B * (H/p) * (W/p), k_pad]`` rows in (channel, dy, dx) order -- the same
    order as a flattened Conv2d kernel, so a stride-p convolution becomes one GEMM.  Columns beyond
    ``C*p*p`` are zero (rows must be a multiple of 16 bytes for the TMA loads)."""
    B, Cc, Hh, Ww = pixel_values.shape
    gh, gw = Hh // patch, Ww // patch
    x = pixel_values[:, :, :gh * patch, :gw * patch].reshape(B, Cc, gh, patch, gw, patch)
    x = x.permute(0, 2, 4, 1, 3, 5).reshape(B * gh * gw, Cc * patch * patch)
    if k_pad > x.shape[1]:
        x = torch.nn.functional.pad(x, (0, k_pad - x.shape[1]))
    return x.contiguous()


def _conv_as_linear(w: torch.Tensor, dev, dtype) -> torch.Tensor:
    w = w.reshape(w.shape[0], -1)
    k_pad = (w.shape[1] + 7) // 8 * 8
    if k_pad != w.shape[1]:
        w = torch.nn.functional.pad(w, (0, k_pad - w.shape[1]))
    return w.to(dev, dtype).contiguous()


# ----------------------------------------------------------------------------- SigLIP
@dataclass
class SiglipConfig:
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_hidden_layers: int = 27
    num_attention_heads: int = 16
    image_size: int = 224
    patch_size: int = 14
    num_channels: int = 3
    layer_norm_eps: float = 1e-6
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_hf(cls, c) -> "SiglipConfig":
        g = (lambda k: c.get(k)) if isinstance(c, dict) else (lambda k: getattr(c, k, None))
        return cls(**{f: g(f) for f in cls.__dataclass_fields__ if g(f) is not None})


class SiglipVisionEncoder:
    """SigLIP vision transformer: ``forward(pixel_values [B,3,H,W])`` -> ``[B, N, hidden]`` after the
    post-LayerNorm, or ``[B, N, proj_dim]`` when a projector (PaliGemma's ``multi_modal_projector``)
    is attached.  All images of a call run as one packed varlen batch.  Heads of 72 are zero-padded
    to 128 so that the attention kernels apply; the softmax scale stays 1/sqrt(72)."""

    def __init__(self, cfg: SiglipConfig, sd: Dict[str, torch.Tensor], *, prefix: str = "vision_model.", device="cuda",
                 dtype=torch.float16, max_images: int = 8, projector: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                 post_norm: bool = True):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        H, heads = cfg.hidden_size, cfg.num_attention_heads
        hd = H // heads
        hd_pad = padded_head_dim(hd)
        g = lambda n: sd[prefix + n]
        self.patch_w = _conv_as_linear(g("embeddings.patch_embedding.weight"), self.device, dtype)
        self.patch_b = g("embeddings.patch_embedding.bias").to(self.device, dtype).contiguous()
        self.pos = g("embeddings.position_embedding.weight").to(self.device, dtype).contiguous()
        self.tokens_per_image = (cfg.image_size // cfg.patch_size) ** 2
        layers = []
        for i in range(cfg.num_hidden_layers):
            b = f"encoder.layers.{i}."
            a = b + "self_attn."
            wqkv, bqkv = fuse_qkv(g(a + "q_proj.weight"), g(a + "k_proj.weight"), g(a + "v_proj.weight"),
                                  g(a + "q_proj.bias"), g(a + "k_proj.bias"), g(a + "v_proj.bias"), heads, hd, hd_pad)
            layers.append(dict(norm1_w=g(b + "layer_norm1.weight"), norm1_b=g(b + "layer_norm1.bias"), wqkv=wqkv, bqkv=bqkv,
                               wo=pad_heads(g(a + "out_proj.weight"), heads, hd, hd_pad, 1), bo=g(a + "out_proj.bias"),
                               norm2_w=g(b + "layer_norm2.weight"), norm2_b=g(b + "layer_norm2.bias"),
                               w_up=g(b + "mlp.fc1.weight"), b_up=g(b + "mlp.fc1.bias"),
                               w_down=g(b + "mlp.fc2.weight"), b_down=g(b + "mlp.fc2.bias")))
        act = {"gelu_pytorch_tanh": "gelu_tanh", "gelu": "gelu_erf"}.get(cfg.hidden_act)
        if act is None:
            raise RPUBackendError(f"unsupported SigLIP activation {cfg.hidden_act}")
        geo = TowerGeometry(H, cfg.num_hidden_layers, heads, hd, cfg.intermediate_size, cfg.layer_norm_eps, act)
        self.tower = VisionTower(geo, layers, max_tokens=max_images * self.tokens_per_image, max_seqs=max_images,
                                 device=device, dtype=dtype)
        self.post_norm = post_norm       # HYViT2 feeds the last block's output straight to its projector
        if post_norm:
            self.post_w = g("post_layernorm.weight").to(self.device, dtype).contiguous()
            self.post_b = g("post_layernorm.bias").to(self.device, dtype).contiguous()
        self.projector = None
        if projector is not None:
            self.projector = tuple(t.to(self.device, dtype).contiguous() for t in projector)

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        B = pixel_values.shape[0]
        n = self.tokens_per_image
        x = patchify(pixel_values.to(self.device, self.dtype), self.cfg.patch_size, self.patch_w.shape[1])
        if x.shape[0] != B * n:
            raise RPUBackendError(f"SigLIP expects {self.cfg.image_size}x{self.cfg.image_size} images")
        hidden = K.gemm(x, self.patch_w, bias=self.patch_b, residual=self.pos.repeat(B, 1) if B > 1 else self.pos)
        self.tower.run(hidden, [n] * B)
        out = K.layernorm(hidden, self.post_w, self.post_b, self.cfg.layer_norm_eps) if self.post_norm else hidden
        if self.projector is not None:
            out = K.gemm(out, self.projector[0], bias=self.projector[1])
        return out.view(B, n, -1)

    __call__ = forward

    def close(self):
        self.tower.close()


# ----------------------------------------------------------------------------- HYViT2
def hyvit2_to_siglip_names(sd: Dict[str, torch.Tensor], layers: int, prefix: str = "") -> Dict[str, torch.Tensor]:
    """timm-style ViT names (``patch_embed.proj``, ``pos_embed``, ``blocks.{i}.norm1 / attn.qkv / attn.proj / norm2 /
    mlp.fc1 / mlp.fc2``) -> the SigLIP names :class:`SiglipVisionEncoder` reads.  The fused ``qkv`` ``[3H, H]`` is split
    into q / k / v; a leading class / register token row of ``pos_embed`` is not expected (HYViT2 has none)."""
    g = lambda n: sd[prefix + n]
    out = {"embeddings.patch_embedding.weight": g("patch_embed.proj.weight"),
           "embeddings.patch_embedding.bias": g("patch_embed.proj.bias")}
    pos = g("pos_embed")
    out["embeddings.position_embedding.weight"] = pos.reshape(-1, pos.shape[-1])
    for i in range(layers):
        b, o = f"blocks.{i}.", f"encoder.layers.{i}."
        qkv_w, qkv_b = g(b + "attn.qkv.weight"), g(b + "attn.qkv.bias")
        H = qkv_w.shape[1]
        for j, n in enumerate(("q_proj", "k_proj", "v_proj")):
            out[o + f"self_attn.{n}.weight"] = qkv_w[j * H:(j + 1) * H]
            out[o + f"self_attn.{n}.bias"] = qkv_b[j * H:(j + 1) * H]
        out[o + "self_attn.out_proj.weight"], out[o + "self_attn.out_proj.bias"] = g(b + "attn.proj.weight"), g(b + "attn.proj.bias")
        for src, dst in (("norm1", "layer_norm1"), ("norm2", "layer_norm2"), ("mlp.fc1", "mlp.fc1"), ("mlp.fc2", "mlp.fc2")):
            out[o + dst + ".weight"], out[o + dst + ".bias"] = g(b + src + ".weight"), g(b + src + ".bias")
    return out


class HYViT2Encoder(SiglipVisionEncoder):
    """HunYuan HYViT2-400M tower: the SigLIP-So400m geometry and block (hidden 1152, 27 layers, 16 heads of 72, MLP 4304,
    LayerScale and drop-path are identities) **without** the post-LayerNorm: the last block's output goes straight to
    the per-token projector, the first linear of the merger (``proj1``); the merger's pooling and second projection stay
    with the caller.  Checkpoints use timm-style names.  Reference: ``src/fused/rpu_hyvit2_vision_model.cpp:1-30``."""

    def __init__(self, cfg: SiglipConfig, sd: Dict[str, torch.Tensor], *, prefix: str = "", device="cuda",
                 dtype=torch.float16, max_images: int = 1, projector: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        mapped = hyvit2_to_siglip_names(sd, cfg.num_hidden_layers, prefix)
        super().__init__(cfg, mapped, prefix="", device=device, dtype=dtype, max_images=max_images, projector=projector,
                         post_norm=False)


# ----------------------------------------------------------------------------- DINOv3
@dataclass
class DINOv3Config:
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    image_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    num_register_tokens: int = 4
    layer_norm_eps: float = 1e-5
    rope_theta: float = 100.0
    hidden_act: str = "gelu"
    use_gated_mlp: bool = False

    @classmethod
    def from_hf(cls, c) -> "DINOv3Config":
        g = (lambda k: c.get(k)) if isinstance(c, dict) else (lambda k: getattr(c, k, None))
        return cls(**{f: g(f) for f in cls.__dataclass_fields__ if g(f) is not None})


class DINOv3Encoder:
    """DINOv3 ViT: ``forward(pixel_values)`` -> ``(last_hidden_state [B, 1+R+N, H], pooled CLS [B, H])``.

    LayerScale is folded into the attention-output and MLP-down projections
    (``gamma * (W x + b) = (gamma * W) x + gamma * b``), so the stack's fused GEMM + residual epilogue
    covers it without a separate multiply.  CLS and register tokens point at the identity row of the
    RoPE table, which is how "rotate the patch tokens only" is expressed."""

    def __init__(self, cfg: DINOv3Config, sd: Dict[str, torch.Tensor], *, prefix: str = "", device="cuda",
                 dtype=torch.float16, max_images: int = 8, max_patches_per_image: Optional[int] = None):
        if cfg.use_gated_mlp:
            raise RPUBackendError("DINOv3 gated-MLP variants are not supported")
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        H, heads = cfg.hidden_size, cfg.num_attention_heads
        hd = H // heads
        hd_pad = padded_head_dim(hd)
        g = lambda n: sd.get(prefix + n)
        self.patch_w = _conv_as_linear(g("embeddings.patch_embeddings.weight"), self.device, dtype)
        self.patch_b = g("embeddings.patch_embeddings.bias").to(self.device, dtype).contiguous()
        self.prefix_tokens = torch.cat((g("embeddings.cls_token")[0], g("embeddings.register_tokens")[0]), 0) \
            .to(self.device, dtype).contiguous()
        self.n_prefix = self.prefix_tokens.shape[0]
        layers = []
        for i in range(cfg.num_hidden_layers):
            b = f"model.layer.{i}." if (prefix + f"model.layer.{i}.norm1.weight") in sd else f"layer.{i}."
            a = b + "attention."
            f32 = lambda n: g(n).float()
            g1, g2 = f32(b + "layer_scale1.lambda1"), f32(b + "layer_scale2.lambda1")
            wqkv, bqkv = fuse_qkv(g(a + "q_proj.weight"), g(a + "k_proj.weight"), g(a + "v_proj.weight"),
                                  g(a + "q_proj.bias"), g(a + "k_proj.bias"), g(a + "v_proj.bias"), heads, hd, hd_pad)
            layers.append(dict(norm1_w=g(b + "norm1.weight"), norm1_b=g(b + "norm1.bias"), wqkv=wqkv, bqkv=bqkv,
                               wo=pad_heads(f32(a + "o_proj.weight") * g1[:, None], heads, hd, hd_pad, 1),
                               bo=f32(a + "o_proj.bias") * g1,
                               norm2_w=g(b + "norm2.weight"), norm2_b=g(b + "norm2.bias"),
                               w_up=g(b + "mlp.up_proj.weight"), b_up=g(b + "mlp.up_proj.bias"),
                               w_down=f32(b + "mlp.down_proj.weight") * g2[:, None], b_down=f32(b + "mlp.down_proj.bias") * g2))
        act = {"gelu": "gelu_erf", "gelu_pytorch_tanh": "gelu_tanh"}.get(cfg.hidden_act)
        if act is None:
            raise RPUBackendError(f"unsupported DINOv3 activation {cfg.hidden_act}")
        geo = TowerGeometry(H, cfg.num_hidden_layers, heads, hd, cfg.intermediate_size, cfg.layer_norm_eps, act)
        per_image = (max_patches_per_image or (cfg.image_size // cfg.patch_size) ** 2) + self.n_prefix
        self.tower = VisionTower(geo, layers, max_tokens=max_images * per_image, max_seqs=max_images, rotary=True,
                                 device=device, dtype=dtype)
        self.norm_w = g("norm.weight").to(self.device, dtype).contiguous()
        self.norm_b = g("norm.bias").to(self.device, dtype).contiguous()
        self.inv_freq = 1.0 / (cfg.rope_theta ** torch.arange(0, 1, 4 / hd, dtype=torch.float32))
        self._geom_cache: Dict[tuple, tuple] = {}

    def _geometry(self, gh: int, gw: int):
        hit = self._geom_cache.get((gh, gw))
        if hit is None:
            rows = [2.0 * ((i + 0.5) / gh) - 1.0 for i in range(gh)]
            cols = [2.0 * ((j + 0.5) / gw) - 1.0 for j in range(gw)]
            cos, sin, axis, ident = rope2d_tables(rows, cols, self.inv_freq, scale=2.0 * math.pi)
            r = torch.arange(gh).view(gh, 1).expand(gh, gw).reshape(-1)
            c = torch.arange(gw).view(1, gw).expand(gh, gw).reshape(-1) + gh
            pos = torch.cat((torch.full((self.n_prefix, 2), ident), torch.stack((r, c), -1)), 0)
            dev = self.device
            hit = (pos.to(dev, torch.int32).contiguous(), cos.to(dev), sin.to(dev), axis.to(dev))
            self._geom_cache[(gh, gw)] = hit
        return hit

    def forward(self, pixel_values: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        B, _, Hh, Ww = pixel_values.shape
        p = self.cfg.patch_size
        gh, gw = Hh // p, Ww // p
        n = gh * gw
        pos, cos, sin, axis = self._geometry(gh, gw)
        x = patchify(pixel_values.to(self.device, self.dtype), p, self.patch_w.shape[1])
        T = self.n_prefix + n
        hidden = torch.empty(B, T, self.cfg.hidden_size, dtype=self.dtype, device=self.device)
        hidden[:, :self.n_prefix] = self.prefix_tokens
        patches = K.gemm(x, self.patch_w, bias=self.patch_b)
        hidden[:, self.n_prefix:] = patches.view(B, n, -1)
        hidden = hidden.view(B * T, -1)
        self.tower.run(hidden, [T] * B, pos=pos.repeat(B, 1) if B > 1 else pos, cos=cos, sin=sin, axis_of_freq=axis)
        out = K.layernorm(hidden, self.norm_w, self.norm_b, self.cfg.layer_norm_eps).view(B, T, -1)
        return out, out[:, 0]

    __call__ = forward

    def close(self):
        self.tower.close()
