"""InternVLA-N1 RGB-D encoder: two DINOv2 ViT-S/14 towers (RGB and depth) and a two-layer perceiver that compresses
their 2 x T x 256 patch tokens into 32 memory tokens for the NavDP head.

    rgb tokens   = DINOv2(normalise(images))          # [B, T * 256, 384]: last block, final LayerNorm, no class token
    depth tokens = DINOv2(depth repeated on 3 channels)
    memory       = [rgb ; depth] + position table
    out          = Linear(TransformerDecoder(queries [32], memory))          # post-LN layers, ReLU, 8 heads of 48

The towers run on the library's ViT stack (LayerScale folded into the attention-output and MLP-down projections, patch
embedding as one GEMM, the 37 x 37 position table resampled to 16 x 16 once at build with DINOv2's bicubic rule); the
perceiver is composed from the GEMM / LayerNorm / attention kernels with heads of 48 on the 64-wide attention kernel.
:class:`TorchRgbdEncoder` is the same computation in plain fp32 PyTorch (``torch.nn.TransformerDecoder`` for the perceiver).

Reference behaviour: ``python/rpu_backend/adapters/internvla_n1/rgbd.py:94-146`` (module layout, preprocessing, token
assembly, tensor names under ``rgbd_encoder.*``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterator, Tuple

import torch
import torch.nn.functional as F

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


@dataclass
class RgbdConfig:
    image_size: int = 224
    patch: int = 14
    hidden: int = 384
    depth: int = 12
    heads: int = 6
    mlp: int = 1536
    pos_grid: int = 37              # side of the checkpoint's position table (518 / 14)
    memory_size: int = 2            # frames
    former_layers: int = 2
    former_heads: int = 8
    former_ff: int = 2048
    embed: int = 384
    eps: float = 1e-6
    former_eps: float = 1e-5

    @property
    def grid(self) -> int:
        return self.image_size // self.patch

    @property
    def queries(self) -> int:
        return self.memory_size * 16


def tiny_rgbd_config(**kw) -> RgbdConfig:
    base = dict(image_size=56, patch=14, hidden=96, depth=2, heads=2, mlp=192, pos_grid=6, memory_size=2, former_heads=2,
                former_ff=128, embed=96)
    base.update(kw)
    return RgbdConfig(**base)


def _tower_shapes(p: str, c: RgbdConfig):
    H = c.hidden
    yield p + "cls_token", (1, 1, H), "embed"
    yield p + "pos_embed", (1, 1 + c.pos_grid ** 2, H), "embed"
    yield p + "patch_embed.proj.weight", (H, 3, c.patch, c.patch), "matrix"
    yield p + "patch_embed.proj.bias", (H,), "bias"
    for i in range(c.depth):
        b = f"{p}blocks.{i}."
        yield b + "norm1.weight", (H,), "norm"
        yield b + "norm1.bias", (H,), "bias"
        yield b + "attn.qkv.weight", (3 * H, H), "matrix"
        yield b + "attn.qkv.bias", (3 * H,), "bias"
        yield b + "attn.proj.weight", (H, H), "matrix"
        yield b + "attn.proj.bias", (H,), "bias"
        yield b + "ls1.gamma", (H,), "norm"
        yield b + "norm2.weight", (H,), "norm"
        yield b + "norm2.bias", (H,), "bias"
        yield b + "mlp.fc1.weight", (c.mlp, H), "matrix"
        yield b + "mlp.fc1.bias", (c.mlp,), "bias"
        yield b + "mlp.fc2.weight", (H, c.mlp), "matrix"
        yield b + "mlp.fc2.bias", (H,), "bias"
        yield b + "ls2.gamma", (H,), "norm"
    yield p + "norm.weight", (H,), "norm"
    yield p + "norm.bias", (H,), "bias"


def rgbd_shapes(c: RgbdConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    H = c.hidden
    yield from _tower_shapes("rgb_model.", c)
    yield from _tower_shapes("depth_model.", c)
    yield "former_query.weight", (c.queries, H), "embed"
    yield "former_pe.weight", (c.memory_size * 2 * c.grid ** 2, H), "embed"
    for i in range(c.former_layers):
        p = f"former_net.layers.{i}."
        for a in ("self_attn", "multihead_attn"):
            yield p + a + ".in_proj_weight", (3 * H, H), "matrix"
            yield p + a + ".in_proj_bias", (3 * H,), "bias"
            yield p + a + ".out_proj.weight", (H, H), "matrix"
            yield p + a + ".out_proj.bias", (H,), "bias"
        yield p + "linear1.weight", (c.former_ff, H), "matrix"
        yield p + "linear1.bias", (c.former_ff,), "bias"
        yield p + "linear2.weight", (H, c.former_ff), "matrix"
        yield p + "linear2.bias", (H,), "bias"
        for n in (1, 2, 3):
            yield p + f"norm{n}.weight", (H,), "norm"
            yield p + f"norm{n}.bias", (H,), "bias"
    yield "project_layer.weight", (c.embed, H), "matrix"
    yield "project_layer.bias", (c.embed,), "bias"


def random_rgbd_state_dict(c: RgbdConfig, *, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in rgbd_shapes(c):
        r = torch.randn(shape, generator=g)
        fan = math.prod(shape[1:]) if len(shape) > 1 else 1
        sd[name] = {"matrix": r / math.sqrt(fan), "embed": r * 0.2, "norm": 1.0 + 0.05 * r, "bias": 0.03 * r}[kind]
    return sd


def resample_pos_embed(pos_embed: torch.Tensor, grid: int, *, offset: float = 0.1) -> torch.Tensor:
    """DINOv2's rule: the patch rows of ``pos_embed [1, 1 + N, H]`` resized bicubically from ``sqrt(N)`` to ``grid`` per side by
    the scale factor ``(grid + offset) / sqrt(N)``; the class row is kept.  Returns ``[1 + grid * grid, H]`` fp32."""
    pe = pos_embed.float()[0]
    n = pe.shape[0] - 1
    side = int(round(math.sqrt(n)))
    if side == grid:
        return pe
    s = float(grid + offset) / side
    patch = pe[1:].reshape(1, side, side, -1).permute(0, 3, 1, 2)
    patch = F.interpolate(patch, scale_factor=(s, s), mode="bicubic", antialias=False)
    if patch.shape[-1] != grid or patch.shape[-2] != grid:
        raise ValueError(f"position table resampled to {tuple(patch.shape[-2:])}, expected {grid} per side")
    return torch.cat((pe[:1], patch.permute(0, 2, 3, 1).reshape(grid * grid, -1)), 0)


def preprocess(images: torch.Tensor, depths: torch.Tensor, size: int):
    """``images [B, T, S, S, 3]`` in [0, 1], ``depths [B, T, S, S, 1]`` -> two ``[B * T, 3, S, S]`` fp32 tensors."""
    mean = torch.tensor(MEAN, device=images.device).view(1, 3, 1, 1)
    std = torch.tensor(STD, device=images.device).view(1, 3, 1, 1)
    ti = (images.float().permute(0, 1, 4, 2, 3).reshape(-1, 3, size, size) - mean) / std
    td = depths.float().permute(0, 1, 4, 2, 3).reshape(-1, 1, size, size).expand(-1, 3, -1, -1).contiguous()
    return ti, td


# ----------------------------------------------------------------------------- fp32 oracle
class TorchRgbdEncoder:
    def __init__(self, c: RgbdConfig, sd: Dict[str, torch.Tensor], device="cpu"):
        self.c, self.device = c, torch.device(device)
        self.sd = {k: v.float().to(self.device) for k, v in sd.items()}
        layer = torch.nn.TransformerDecoderLayer(c.hidden, c.former_heads, c.former_ff, dropout=0.0, batch_first=True,
                                                 layer_norm_eps=c.former_eps)
        self.former = torch.nn.TransformerDecoder(layer, c.former_layers).to(self.device).eval()
        self.former.load_state_dict({k[len("former_net."):]: v for k, v in self.sd.items() if k.startswith("former_net.")})

    @torch.no_grad()
    def tower(self, p: str, x: torch.Tensor) -> torch.Tensor:
        c, sd, H = self.c, self.sd, self.c.hidden
        B = x.shape[0]
        t = F.conv2d(x, sd[p + "patch_embed.proj.weight"], sd[p + "patch_embed.proj.bias"], stride=c.patch).flatten(2).transpose(1, 2)
        t = torch.cat((sd[p + "cls_token"].expand(B, -1, -1), t), 1) + resample_pos_embed(sd[p + "pos_embed"], c.grid).to(self.device)[None]
        hd = H // c.heads
        for i in range(c.depth):
            b = f"{p}blocks.{i}."
            n = F.layer_norm(t, (H,), sd[b + "norm1.weight"], sd[b + "norm1.bias"], c.eps)
            q, k, v = F.linear(n, sd[b + "attn.qkv.weight"], sd[b + "attn.qkv.bias"]).chunk(3, -1)
            sp = lambda z: z.reshape(B, -1, c.heads, hd).transpose(1, 2)
            a = F.scaled_dot_product_attention(sp(q), sp(k), sp(v)).transpose(1, 2).reshape(B, -1, H)
            t = t + sd[b + "ls1.gamma"] * F.linear(a, sd[b + "attn.proj.weight"], sd[b + "attn.proj.bias"])
            n = F.layer_norm(t, (H,), sd[b + "norm2.weight"], sd[b + "norm2.bias"], c.eps)
            m = F.linear(F.gelu(F.linear(n, sd[b + "mlp.fc1.weight"], sd[b + "mlp.fc1.bias"])), sd[b + "mlp.fc2.weight"], sd[b + "mlp.fc2.bias"])
            t = t + sd[b + "ls2.gamma"] * m
        return F.layer_norm(t, (H,), sd[p + "norm.weight"], sd[p + "norm.bias"], c.eps)[:, 1:]

    @torch.no_grad()
    def forward(self, images: torch.Tensor, depths: torch.Tensor) -> torch.Tensor:
        c, sd = self.c, self.sd
        B, T = images.shape[0], images.shape[1]
        ti, td = preprocess(images.to(self.device), depths.to(self.device), c.image_size)
        it = self.tower("rgb_model.", ti).reshape(B, T * c.grid ** 2, -1)
        dt = self.tower("depth_model.", td).reshape(B, T * c.grid ** 2, -1)
        mem = torch.cat((it, dt), 1) + sd["former_pe.weight"][None, :2 * T * c.grid ** 2]
        q = sd["former_query.weight"][None].expand(B, -1, -1)
        return F.linear(self.former(q, mem), sd["project_layer.weight"], sd["project_layer.bias"])

    __call__ = forward


# ----------------------------------------------------------------------------- device engine
class RgbdEncoder:
    """``forward(images [B, T, S, S, 3], depths [B, T, S, S, 1]) -> rgbd_embed [B, 32, embed]`` (fp32, on the device)."""

    def __init__(self, c: RgbdConfig, sd: Dict[str, torch.Tensor], *, max_batch: int = 1, device="cuda", dtype=torch.float16):
        from ..ops import kernels as K
        from ..runtime.stack import pad_heads
        from .vision import TowerGeometry, VisionTower, _conv_as_linear, fuse_qkv, padded_head_dim
        bad = [f"{n}: {tuple(sd[n].shape) if n in sd else 'missing'}, expected {s}" for n, s, _ in rgbd_shapes(c)
               if n not in sd or tuple(sd[n].shape) != s]
        if bad:
            raise ValueError(f"RGB-D encoder weights do not fit the profile ({len(bad)} tensors): " + "; ".join(bad[:5]))
        self.K, self.c, self.device, self.dtype, self.B = K, c, torch.device(device), dtype, max_batch
        dev, H, hd = self.device, c.hidden, c.hidden // c.heads
        hp = padded_head_dim(hd)
        t = lambda w: w.to(dev, dtype).contiguous()
        n_img = max_batch * c.memory_size
        per = 1 + c.grid ** 2
        self.towers = {}
        for p in ("rgb_model.", "depth_model."):
            layers = []
            for i in range(c.depth):
                b = f"{p}blocks.{i}."
                w, bias = sd[b + "attn.qkv.weight"], sd[b + "attn.qkv.bias"]
                g1, g2 = sd[b + "ls1.gamma"].float(), sd[b + "ls2.gamma"].float()
                wqkv, bqkv = fuse_qkv(w[:H], w[H:2 * H], w[2 * H:], bias[:H], bias[H:2 * H], bias[2 * H:], c.heads, hd, hp)
                layers.append(dict(norm1_w=sd[b + "norm1.weight"], norm1_b=sd[b + "norm1.bias"], wqkv=wqkv, bqkv=bqkv,
                                   wo=pad_heads(sd[b + "attn.proj.weight"].float() * g1[:, None], c.heads, hd, hp, 1),
                                   bo=sd[b + "attn.proj.bias"].float() * g1,
                                   norm2_w=sd[b + "norm2.weight"], norm2_b=sd[b + "norm2.bias"],
                                   w_up=sd[b + "mlp.fc1.weight"], b_up=sd[b + "mlp.fc1.bias"],
                                   w_down=sd[b + "mlp.fc2.weight"].float() * g2[:, None], b_down=sd[b + "mlp.fc2.bias"].float() * g2))
            geo = TowerGeometry(H, c.depth, c.heads, hd, c.mlp, c.eps, "gelu_erf")
            tower = VisionTower(geo, layers, max_tokens=n_img * per, max_seqs=n_img, rotary=False, device=device, dtype=dtype)
            pos = resample_pos_embed(sd[p + "pos_embed"], c.grid)
            self.towers[p] = dict(tower=tower, patch_w=_conv_as_linear(sd[p + "patch_embed.proj.weight"], dev, dtype),
                                  patch_b=t(sd[p + "patch_embed.proj.bias"]),
                                  cls=t(sd[p + "cls_token"].float()[0] + pos[:1]), pos=t(pos[1:]),
                                  norm_w=t(sd[p + "norm.weight"]), norm_b=t(sd[p + "norm.bias"]))
        # perceiver (post-LN decoder layers)
        fh, fhd = c.former_heads, H // c.former_heads
        self.fhp = padded_head_dim(fhd)
        self.fhd, self.FD = fhd, fh * self.fhp
        pack = lambda w: K.pack_weight(t(w))
        self.former = []
        for i in range(c.former_layers):
            p = f"former_net.layers.{i}."
            L = {}
            for a, tag in (("self_attn", "s"), ("multihead_attn", "c")):
                w, b = sd[p + a + ".in_proj_weight"], sd[p + a + ".in_proj_bias"]
                ws = [pad_heads(w[j * H:(j + 1) * H], fh, fhd, self.fhp, 0) for j in range(3)]
                bs = [pad_heads(b[j * H:(j + 1) * H], fh, fhd, self.fhp, 0) for j in range(3)]
                if tag == "s":
                    L["s_qkv_w"], L["s_qkv_b"] = pack(torch.cat(ws, 0)), t(torch.cat(bs, 0))
                else:
                    L["c_q_w"], L["c_q_b"] = pack(ws[0]), t(bs[0])
                    L["c_kv_w"], L["c_kv_b"] = pack(torch.cat(ws[1:], 0)), t(torch.cat(bs[1:], 0))
                L[tag + "_o_w"] = pack(pad_heads(sd[p + a + ".out_proj.weight"], fh, fhd, self.fhp, 1))
                L[tag + "_o_b"] = t(sd[p + a + ".out_proj.bias"])
            L["ff1_w"], L["ff1_b"] = pack(sd[p + "linear1.weight"]), t(sd[p + "linear1.bias"])
            L["ff2_w"], L["ff2_b"] = pack(sd[p + "linear2.weight"]), t(sd[p + "linear2.bias"])
            for n in (1, 2, 3):
                L[f"n{n}_w"], L[f"n{n}_b"] = t(sd[p + f"norm{n}.weight"]), t(sd[p + f"norm{n}.bias"])
            self.former.append(L)
        self.query = t(sd["former_query.weight"])
        self.pe = t(sd["former_pe.weight"])
        self.proj_w, self.proj_b = pack(sd["project_layer.weight"]), t(sd["project_layer.bias"])
        self.mean = torch.tensor(MEAN, device=dev).view(1, 3, 1, 1)
        self.std = torch.tensor(STD, device=dev).view(1, 3, 1, 1)
        self.status = torch.zeros(32, dtype=torch.int32, device=dev)

    def _tower(self, p: str, x: torch.Tensor) -> torch.Tensor:
        """``x [N, 3, S, S]`` -> patch tokens ``[N, grid^2, H]`` after the final LayerNorm."""
        from .vision import patchify
        K, c, tw = self.K, self.c, self.towers[p]
        N, n, H = x.shape[0], c.grid ** 2, c.hidden
        patches = K.gemm(patchify(x.to(self.dtype), c.patch, tw["patch_w"].shape[1]), tw["patch_w"], bias=tw["patch_b"],
                         residual=tw["pos"].repeat(N, 1))
        hidden = torch.empty(N, 1 + n, H, dtype=self.dtype, device=self.device)
        hidden[:, 0] = tw["cls"]
        hidden[:, 1:] = patches.view(N, n, H)
        hidden = hidden.view(N * (1 + n), H)
        tw["tower"].run(hidden, [1 + n] * N)
        return K.layernorm(hidden, tw["norm_w"], tw["norm_b"], c.eps).view(N, 1 + n, H)[:, 1:]

    @torch.no_grad()
    def forward(self, images: torch.Tensor, depths: torch.Tensor) -> torch.Tensor:
        K, c, dev, H = self.K, self.c, self.device, self.c.hidden
        B, T = images.shape[0], images.shape[1]
        if B > self.B or T != c.memory_size or tuple(images.shape[2:]) != (c.image_size, c.image_size, 3):
            raise ValueError(f"images must be [<= {self.B}, {c.memory_size}, {c.image_size}, {c.image_size}, 3], got {tuple(images.shape)}")
        ti, td = preprocess(images.to(dev), depths.to(dev), c.image_size)
        n = c.grid ** 2
        M = 2 * T * n
        mem = torch.empty(B, M, H, dtype=self.dtype, device=dev)
        mem[:, :T * n] = self._tower("rgb_model.", ti).reshape(B, T * n, H)
        mem[:, T * n:] = self._tower("depth_model.", td).reshape(B, T * n, H)
        mem.add_(self.pe[None, :M])
        mem = mem.view(B * M, H)
        Q, FD, fh = c.queries, self.FD, c.former_heads
        x = self.query.repeat(B, 1)                                            # [B * Q, H]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        q_start, q_len = i32([b * Q for b in range(B)]), i32([Q] * B)
        m_start, m_len = i32([b * M for b in range(B)]), i32([M] * B)
        scale = 1.0 / math.sqrt(self.fhd)
        att = torch.empty(B * Q, FD, dtype=self.dtype, device=dev)
        for L in self.former:
            qkv = K.gemm(x, L["s_qkv_w"], packed_shape=(3 * FD, H), bias=L["s_qkv_b"])
            K.attention_prefill(qkv[:, :FD], att, Hq=fh, Hkv=fh, hd=self.fhp, q_start=q_start, q_len=q_len, kv_len=q_len, max_q_len=Q,
                                k=qkv[:, FD:2 * FD], v=qkv[:, 2 * FD:], kv_start=q_start, causal=False, scale=scale, status=self.status,
                                max_kv_len=Q)
            y = K.gemm(att, L["s_o_w"], packed_shape=(H, FD), bias=L["s_o_b"], residual=x)
            x = K.layernorm(y, L["n1_w"], L["n1_b"], c.former_eps)
            q = K.gemm(x, L["c_q_w"], packed_shape=(FD, H), bias=L["c_q_b"])
            kv = K.gemm(mem, L["c_kv_w"], packed_shape=(2 * FD, H), bias=L["c_kv_b"])
            K.attention_prefill(q, att, Hq=fh, Hkv=fh, hd=self.fhp, q_start=q_start, q_len=q_len, kv_len=m_len, max_q_len=Q,
                                k=kv[:, :FD], v=kv[:, FD:], kv_start=m_start, causal=False, scale=scale, status=self.status)
            y = K.gemm(att, L["c_o_w"], packed_shape=(H, FD), bias=L["c_o_b"], residual=x)
            x = K.layernorm(y, L["n2_w"], L["n2_b"], c.former_eps)
            f = K.gemm(x, L["ff1_w"], packed_shape=(c.former_ff, H), bias=L["ff1_b"]).clamp_min_(0.0)
            y = K.gemm(f, L["ff2_w"], packed_shape=(H, c.former_ff), bias=L["ff2_b"], residual=x)
            x = K.layernorm(y, L["n3_w"], L["n3_b"], c.former_eps)
        out = K.gemm(x, self.proj_w, packed_shape=(c.embed, H), bias=self.proj_b)
        return out.float().view(B, Q, c.embed)

    __call__ = forward

    def check_status(self) -> None:
        torch.cuda.synchronize()
        st = self.status.tolist()
        if st[0] != 0:
            from ..runtime.errors import RPUBackendError
            raise RPUBackendError(f"device status {st[:4]} (code, block, kernel, detail)")

    def close(self) -> None:
        for tw in self.towers.values():
            tw["tower"].close()


__all__ = ["RgbdConfig", "RgbdEncoder", "TorchRgbdEncoder", "tiny_rgbd_config", "rgbd_shapes", "random_rgbd_state_dict",
           "resample_pos_embed", "preprocess"]
