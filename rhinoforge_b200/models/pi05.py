"""Pi0.5 vision-language-action policy: SigLIP + PaliGemma (Gemma-2B) prefix + adaRMS action expert.

Data flow of one ``predict_action_chunk``:

  images [n_views,3,224,224] -> SigLIP -> projector          \\
  language tokens -> embedding * sqrt(width)                   > prefix rows -> Gemma-2B, bidirectional,
                                                              /   K/V of every layer into the paged cache
  noise x_1 [horizon, action_dim]; for s in 0..num_steps-1 (t_s = 1 + s*dt, dt = -1/num_steps):
      h = action_in_proj(x)                                   action expert (Gemma-300M geometry):
      per layer: adaRMS(h | t_s) -> qkv -> RoPE at prefix_len + i -> K/V written behind the prefix
                 attention over [prefix | all action rows] -> o_proj -> h += gate * o
                 adaRMS -> GeGLU MLP -> h += gate * mlp
      v = action_out_proj(adaRMS_final(h | t_s));  x <- x + dt * v

Only valid prefix rows are packed (missing cameras and language padding are simply absent), which is
the same computation as the padded/masked formulation: masked rows never contribute and positions are
the running count of valid rows.  The adaRMS modulation ``dense(cond_s)`` depends on the time step
alone, so all ``[scale | shift | gate]`` vectors of all layers and steps are computed once per
``num_steps`` and the denoise loop contains no conditioning GEMV at all; ``dt`` is folded into the
output projection so the Euler update is that GEMM's residual epilogue.  The whole loop replays from
one CUDA graph.

Reference behaviour: ``python/rpu_backend/adapters/pi05/runtime.py:448-620`` (prefix build, masks),
``adapters/pi05/weights.py:176-220`` (conditioning schedule), ``adapters/pi05/adarms.py:43-118``,
``src/fused/rpu_gemma_model.cpp:688-955``, ``src/fused/rpu_adarms_model.cpp:1-33``,
``src/fused/rpu_pi05_denoise_step_model.cpp:453-526,661-1075`` (step body, Euler unroll).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Dict, Iterator, Sequence, Tuple

import torch
import torch.nn.functional as F

from .vision import SiglipConfig


@dataclass
class GemmaGeometry:
    hidden: int
    inter: int
    layers: int = 18
    heads: int = 8
    kv_heads: int = 1
    head_dim: int = 256
    eps: float = 1e-6
    rope_theta: float = 10000.0


@dataclass
class Pi05Config:
    vlm: GemmaGeometry = field(default_factory=lambda: GemmaGeometry(2048, 16384))
    expert: GemmaGeometry = field(default_factory=lambda: GemmaGeometry(1024, 4096))
    vision: SiglipConfig = field(default_factory=SiglipConfig)
    vocab_size: int = 257152
    action_dim: int = 32
    horizon: int = 50
    min_period: float = 4e-3
    max_period: float = 4.0
    max_lang_tokens: int = 200
    num_views: int = 3

    @property
    def tokens_per_image(self) -> int:
        return (self.vision.image_size // self.vision.patch_size) ** 2


def tiny_pi05_config() -> Pi05Config:
    return Pi05Config(vlm=GemmaGeometry(128, 256, layers=3, heads=2, kv_heads=1, head_dim=64),
                      expert=GemmaGeometry(64, 128, layers=3, heads=2, kv_heads=1, head_dim=64),
                      vision=SiglipConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                          num_attention_heads=2, image_size=56, patch_size=14),
                      vocab_size=512, action_dim=8, horizon=10, max_lang_tokens=16, num_views=2)


VLM = "paligemma_with_expert.paligemma.model."
EXP = "paligemma_with_expert.gemma_expert.model."


def pi05_weight_shapes(cfg: Pi05Config) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """(checkpoint name, shape, kind) of every tensor; kind in {matrix, norm, bias}."""
    v = cfg.vision
    vp = VLM + "vision_tower.vision_model."
    yield vp + "embeddings.patch_embedding.weight", (v.hidden_size, v.num_channels, v.patch_size, v.patch_size), "matrix"
    yield vp + "embeddings.patch_embedding.bias", (v.hidden_size,), "bias"
    yield vp + "embeddings.position_embedding.weight", (cfg.tokens_per_image, v.hidden_size), "matrix"
    for i in range(v.num_hidden_layers):
        b = f"{vp}encoder.layers.{i}."
        for n in ("layer_norm1", "layer_norm2"):
            yield b + n + ".weight", (v.hidden_size,), "norm1"
            yield b + n + ".bias", (v.hidden_size,), "bias"
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            yield b + f"self_attn.{n}.weight", (v.hidden_size, v.hidden_size), "matrix"
            yield b + f"self_attn.{n}.bias", (v.hidden_size,), "bias"
        yield b + "mlp.fc1.weight", (v.intermediate_size, v.hidden_size), "matrix"
        yield b + "mlp.fc1.bias", (v.intermediate_size,), "bias"
        yield b + "mlp.fc2.weight", (v.hidden_size, v.intermediate_size), "matrix"
        yield b + "mlp.fc2.bias", (v.hidden_size,), "bias"
    yield vp + "post_layernorm.weight", (v.hidden_size,), "norm1"
    yield vp + "post_layernorm.bias", (v.hidden_size,), "bias"
    yield VLM + "multi_modal_projector.linear.weight", (cfg.vlm.hidden, v.hidden_size), "matrix"
    yield VLM + "multi_modal_projector.linear.bias", (cfg.vlm.hidden,), "bias"
    yield VLM + "language_model.embed_tokens.weight", (cfg.vocab_size, cfg.vlm.hidden), "matrix"
    for pre, g, ada in ((VLM + "language_model.", cfg.vlm, False), (EXP, cfg.expert, True)):
        for i in range(g.layers):
            b = f"{pre}layers.{i}."
            yield b + "self_attn.q_proj.weight", (g.heads * g.head_dim, g.hidden), "matrix"
            yield b + "self_attn.k_proj.weight", (g.kv_heads * g.head_dim, g.hidden), "matrix"
            yield b + "self_attn.v_proj.weight", (g.kv_heads * g.head_dim, g.hidden), "matrix"
            yield b + "self_attn.o_proj.weight", (g.hidden, g.heads * g.head_dim), "matrix"
            yield b + "mlp.gate_proj.weight", (g.inter, g.hidden), "matrix"
            yield b + "mlp.up_proj.weight", (g.inter, g.hidden), "matrix"
            yield b + "mlp.down_proj.weight", (g.hidden, g.inter), "matrix"
            for n in ("input_layernorm", "post_attention_layernorm"):
                if ada:
                    yield b + n + ".dense.weight", (3 * g.hidden, g.hidden), "matrix"
                    yield b + n + ".dense.bias", (3 * g.hidden,), "bias"
                else:
                    yield b + n + ".weight", (g.hidden,), "norm0"
        if ada:
            yield pre + "norm.dense.weight", (3 * g.hidden, g.hidden), "matrix"
            yield pre + "norm.dense.bias", (3 * g.hidden,), "bias"
        else:
            yield pre + "norm.weight", (g.hidden,), "norm0"
    e = cfg.expert.hidden
    yield "action_in_proj.weight", (e, cfg.action_dim), "matrix"
    yield "action_in_proj.bias", (e,), "bias"
    yield "action_out_proj.weight", (cfg.action_dim, e), "matrix"
    yield "action_out_proj.bias", (cfg.action_dim,), "bias"
    for n in ("time_mlp_in", "time_mlp_out"):
        yield n + ".weight", (e, e), "matrix"
        yield n + ".bias", (e,), "bias"


def random_pi05_state_dict(cfg: Pi05Config, *, seed: int = 0, std: float = 0.02, dtype=torch.float16,
                           device="cpu") -> Dict[str, torch.Tensor]:
    """Random-init weights of the real architecture (synthetic benchmarks and tests)."""
    gen_dev = "cuda" if str(device).startswith("cuda") else "cpu"     # full-size models are drawn on the device
    g = torch.Generator(device=gen_dev).manual_seed(seed)
    sd = {}
    for name, shape, kind in pi05_weight_shapes(cfg):
        r = torch.randn(shape, generator=g, device=gen_dev)
        if kind == "matrix":
            t = r * std
        elif kind == "norm1":
            t = 1.0 + 0.05 * r
        elif kind == "norm0":                       # Gemma stores (w - 1)
            t = 0.05 * r
        else:
            t = 0.02 * r
        sd[name] = t.to(device, dtype)
    return sd


def sinusoidal_time_embedding(t: torch.Tensor, dim: int, min_period: float, max_period: float) -> torch.Tensor:
    """``[n] -> [n, dim]``: sin | cos over ``dim/2`` log-spaced periods in ``[min_period, max_period]`` (fp64 math)."""
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64)
    period = min_period * (max_period / min_period) ** frac
    ang = (2.0 * math.pi / period)[None, :] * t.double()[:, None]
    return torch.cat((ang.sin(), ang.cos()), 1)


def conditioning_schedule(sd, cfg: Pi05Config, num_steps: int) -> torch.Tensor:
    """``cond_all [num_steps, expert_hidden]`` (fp32): ``silu(W2 silu(W1 sincos(t_s)))`` with ``t_s = 1 + s*dt``."""
    dt = -1.0 / num_steps
    ts = torch.tensor([1.0 + s * dt for s in range(num_steps)], dtype=torch.float32)
    emb = sinusoidal_time_embedding(ts, cfg.expert.hidden, cfg.min_period, cfg.max_period).float()
    dev = sd["time_mlp_in.weight"].device
    x = F.silu(F.linear(emb.to(dev), sd["time_mlp_in.weight"].float(), sd["time_mlp_in.bias"].float()))
    return F.silu(F.linear(x, sd["time_mlp_out.weight"].float(), sd["time_mlp_out.bias"].float()))


# ----------------------------------------------------------------------------- fp32 oracle
class TorchPi05:
    """Plain PyTorch implementation (any dtype/device) of the same computation, written in the padded /
    masked formulation so that it checks the packed formulation of :class:`Pi05Engine` independently."""

    def __init__(self, cfg: Pi05Config, sd: Dict[str, torch.Tensor], *, dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.sd = {k: v.to(self.device, dtype) for k, v in sd.items()}

    # -- SigLIP + projector
    def embed_images(self, images: torch.Tensor) -> torch.Tensor:
        cfg, sd, v = self.cfg, self.sd, self.cfg.vision
        vp = VLM + "vision_tower.vision_model."
        x = F.conv2d(images.to(self.device, self.dtype), sd[vp + "embeddings.patch_embedding.weight"],
                     sd[vp + "embeddings.patch_embedding.bias"], stride=v.patch_size)
        x = x.flatten(2).transpose(1, 2) + sd[vp + "embeddings.position_embedding.weight"]
        heads, hd = v.num_attention_heads, v.hidden_size // v.num_attention_heads
        act = (lambda t: F.gelu(t, approximate="tanh")) if v.hidden_act == "gelu_pytorch_tanh" else F.gelu
        for i in range(v.num_hidden_layers):
            b = f"{vp}encoder.layers.{i}."
            h = F.layer_norm(x, (v.hidden_size,), sd[b + "layer_norm1.weight"], sd[b + "layer_norm1.bias"], v.layer_norm_eps)
            q, k, vv = (F.linear(h, sd[b + f"self_attn.{n}_proj.weight"], sd[b + f"self_attn.{n}_proj.bias"])
                        .view(x.shape[0], -1, heads, hd).transpose(1, 2) for n in "qkv")
            a = torch.softmax((q.float() @ k.float().transpose(-1, -2)) / math.sqrt(hd), -1) @ vv.float()
            a = a.to(self.dtype).transpose(1, 2).reshape(x.shape[0], -1, v.hidden_size)
            x = x + F.linear(a, sd[b + "self_attn.out_proj.weight"], sd[b + "self_attn.out_proj.bias"])
            h = F.layer_norm(x, (v.hidden_size,), sd[b + "layer_norm2.weight"], sd[b + "layer_norm2.bias"], v.layer_norm_eps)
            x = x + F.linear(act(F.linear(h, sd[b + "mlp.fc1.weight"], sd[b + "mlp.fc1.bias"])),
                             sd[b + "mlp.fc2.weight"], sd[b + "mlp.fc2.bias"])
        x = F.layer_norm(x, (v.hidden_size,), sd[vp + "post_layernorm.weight"], sd[vp + "post_layernorm.bias"], v.layer_norm_eps)
        return F.linear(x, sd[VLM + "multi_modal_projector.linear.weight"], sd[VLM + "multi_modal_projector.linear.bias"])

    @staticmethod
    def _rms(x, eps):
        xf = x.float()
        return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)

    def _rope(self, t, pos, g: GemmaGeometry):           # t [B, H, S, hd], pos [B, S]
        inv = 1.0 / (g.rope_theta ** (torch.arange(0, g.head_dim, 2, dtype=torch.float32, device=self.device) / g.head_dim))
        ang = pos.float()[:, None, :, None] * inv
        cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)
        h = t.shape[-1] // 2
        rot = torch.cat((-t[..., h:], t[..., :h]), -1)
        return (t.float() * cos + rot.float() * sin).to(t.dtype)

    def _layer(self, pre, i, g, x, pos, mask, past_kv, cond):
        """One Gemma layer over rows ``x`` [B,S,H]; K/V are appended to ``past_kv`` (or start it)."""
        sd, b = self.sd, f"{pre}layers.{i}."
        B, S, _ = x.shape

        def norm(name, t):
            n = self._rms(t, g.eps)
            if cond is None:
                return (n * (1.0 + sd[b + name + ".weight"].float())).to(self.dtype), None
            mod = F.linear(cond, sd[b + name + ".dense.weight"], sd[b + name + ".dense.bias"]).float()
            sc, sh, gate = mod.chunk(3, -1)
            return (n * (1.0 + sc[:, None]) + sh[:, None]).to(self.dtype), gate[:, None].to(self.dtype)

        h, gate = norm("input_layernorm", x)
        q = F.linear(h, sd[b + "self_attn.q_proj.weight"]).view(B, S, g.heads, g.head_dim).transpose(1, 2)
        k = F.linear(h, sd[b + "self_attn.k_proj.weight"]).view(B, S, g.kv_heads, g.head_dim).transpose(1, 2)
        v = F.linear(h, sd[b + "self_attn.v_proj.weight"]).view(B, S, g.kv_heads, g.head_dim).transpose(1, 2)
        q, k = self._rope(q, pos, g), self._rope(k, pos, g)
        if past_kv is not None:
            k, v = torch.cat((past_kv[0], k), 2), torch.cat((past_kv[1], v), 2)
        G = g.heads // g.kv_heads
        if self.dtype != torch.float32:      # 16-bit baseline runs: the library's fused attention
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask[:, None], enable_gqa=True)
        else:
            s = (q.float() @ k.repeat_interleave(G, 1).float().transpose(-1, -2)) / math.sqrt(g.head_dim)
            s = s.masked_fill(~mask[:, None], float("-inf"))
            a = (torch.softmax(s, -1) @ v.repeat_interleave(G, 1).float()).to(self.dtype)
        o = F.linear(a.transpose(1, 2).reshape(B, S, -1), sd[b + "self_attn.o_proj.weight"])
        x = x + (o if gate is None else gate * o)
        h, gate = norm("post_attention_layernorm", x)
        m = F.gelu(F.linear(h, sd[b + "mlp.gate_proj.weight"]), approximate="tanh") * F.linear(h, sd[b + "mlp.up_proj.weight"])
        m = F.linear(m, sd[b + "mlp.down_proj.weight"])
        return x + (m if gate is None else gate * m), (k, v)

    @torch.no_grad()
    def prefix(self, images: torch.Tensor, image_mask: torch.Tensor, tokens: torch.Tensor, token_mask: torch.Tensor):
        """images [B,V,3,H,W], image_mask [B,V] bool, tokens [B,L], token_mask [B,L] bool ->
        (per-layer (K,V) over padded prefix rows, pad mask [B,P])."""
        cfg = self.cfg
        B, V = images.shape[:2]
        img = self.embed_images(images.flatten(0, 1)).view(B, V * cfg.tokens_per_image, -1)
        lang = F.embedding(tokens.to(self.device), self.sd[VLM + "language_model.embed_tokens.weight"]) * math.sqrt(cfg.vlm.hidden)
        x = torch.cat((img, lang.to(self.dtype)), 1)
        pad = torch.cat((image_mask.to(self.device)[:, :, None].expand(B, V, cfg.tokens_per_image).reshape(B, -1),
                         token_mask.to(self.device)), 1).bool()
        pos = pad.long().cumsum(1) - 1
        mask = pad[:, None, :] & pad[:, :, None]                      # bidirectional over valid rows
        mask = mask | torch.eye(pad.shape[1], dtype=torch.bool, device=self.device)[None]   # keep pad rows finite
        kvs = []
        for i in range(cfg.vlm.layers):
            x, kv = self._layer(VLM + "language_model.", i, cfg.vlm, x, pos.clamp(min=0), mask, None, None)
            kvs.append(kv)
        return kvs, pad

    @torch.no_grad()
    def sample_actions(self, images, image_mask, tokens, token_mask, noise: torch.Tensor, num_steps: int = 10) -> torch.Tensor:
        """noise [B, horizon, action_dim] -> actions of the same shape (fp32 Euler integration from t=1 to 0)."""
        cfg, sd = self.cfg, self.sd
        kvs, pad = self.prefix(images, image_mask, tokens, token_mask)
        B, P = pad.shape
        n = cfg.horizon
        cond_all = conditioning_schedule(sd, cfg, num_steps).to(self.device, self.dtype)
        x = noise.to(self.device, self.dtype)
        dt = -1.0 / num_steps
        pos = pad.long().sum(1, keepdim=True) + torch.arange(n, device=self.device)[None]
        mask = torch.cat((pad[:, None, :].expand(B, n, P), torch.ones(B, n, n, dtype=torch.bool, device=self.device)), 2)
        for s in range(num_steps):
            cond = cond_all[s][None].expand(B, -1)
            h = F.linear(x, sd["action_in_proj.weight"], sd["action_in_proj.bias"])
            for i in range(cfg.expert.layers):
                h, _ = self._layer(EXP, i, cfg.expert, h, pos, mask, kvs[i], cond)
            mod = F.linear(cond, sd[EXP + "norm.dense.weight"], sd[EXP + "norm.dense.bias"]).float()
            sc, sh, _ = mod.chunk(3, -1)
            hn = (self._rms(h, cfg.expert.eps) * (1.0 + sc[:, None]) + sh[:, None]).to(self.dtype)
            v = F.linear(hn, sd["action_out_proj.weight"], sd["action_out_proj.bias"])
            x = x + dt * v
        return x


# ----------------------------------------------------------------------------- device engine
class Pi05Engine:
    """Pi0.5 on the accelerator: packed-prefix prefill + CUDA-graph denoise loop.

    ``predict(images, image_mask, tokens, token_mask, noise, num_steps)`` returns ``[B, horizon, action_dim]``.
    The result tensor is a stable buffer that the next call overwrites: copy what you keep."""

    def __init__(self, cfg: Pi05Config, sd: Dict[str, torch.Tensor], *, device="cuda", dtype=torch.float16,
                 max_batch: int = 1):
        from ..ops import kernels as K
        from ..runtime.kv_cache import PagedKV
        from ..runtime.stack import NativeStack, StackSpec
        from .vision import SiglipVisionEncoder
        self.K = K
        self.cfg, self.device, self.dtype, self.max_batch = cfg, torch.device(device), dtype, max_batch
        g = lambda n: sd[n]
        dev = self.device
        self.vision = SiglipVisionEncoder(cfg.vision, sd, prefix=VLM + "vision_tower.vision_model.", device=device,
                                          dtype=dtype, max_images=max_batch * cfg.num_views,
                                          projector=(g(VLM + "multi_modal_projector.linear.weight"),
                                                     g(VLM + "multi_modal_projector.linear.bias")))
        self.embed = g(VLM + "language_model.embed_tokens.weight").to(dev, dtype).contiguous()
        self.max_prefix = cfg.num_views * cfg.tokens_per_image + cfg.max_lang_tokens
        self.max_seq = (self.max_prefix + cfg.horizon + 15) // 16 * 16
        v, e = cfg.vlm, cfg.expert
        if (v.layers, v.kv_heads, v.head_dim) != (e.layers, e.kv_heads, e.head_dim):
            raise ValueError("prefix LM and action expert must share the KV geometry (layers, kv heads, head_dim)")
        self.cache = PagedKV(v.layers, max_batch, self.max_seq, v.kv_heads, v.head_dim, device=device, dtype=dtype)
        self.cache.reserve_all()

        def layers_of(pre, geo, ada):
            out = []
            for i in range(geo.layers):
                b = f"{pre}layers.{i}."
                d = dict(wqkv=torch.cat([g(b + f"self_attn.{n}_proj.weight") for n in "qkv"], 0),
                         wo=g(b + "self_attn.o_proj.weight"),
                         w_up=torch.cat((g(b + "mlp.gate_proj.weight"), g(b + "mlp.up_proj.weight")), 0),
                         w_down=g(b + "mlp.down_proj.weight"))
                if not ada:
                    d["norm1_w"], d["norm2_w"] = g(b + "input_layernorm.weight"), g(b + "post_attention_layernorm.weight")
                out.append(d)
            return out

        common = dict(mlp="geglu_tanh", paged_kv=True, causal=False)
        self.prefix_stack = NativeStack(
            StackSpec(layers=v.layers, hidden=v.hidden, heads=v.heads, kv_heads=v.kv_heads, head_dim=v.head_dim,
                      inter=v.inter, norm="rms_gemma", eps=v.eps, rot_dim=v.head_dim,
                      max_tokens=max_batch * self.max_prefix, max_seqs=max_batch, **common),
            layers_of(VLM + "language_model.", v, False), device=device, dtype=dtype, kv_cache=self.cache)
        self.expert_stack = NativeStack(
            StackSpec(layers=e.layers, hidden=e.hidden, heads=e.heads, kv_heads=e.kv_heads, head_dim=e.head_dim,
                      inter=e.inter, norm="adarms", eps=e.eps, rot_dim=e.head_dim, gated_residual=True,
                      max_tokens=max_batch * cfg.horizon, max_seqs=max_batch * cfg.horizon, **common),
            layers_of(EXP, e, True), device=device, dtype=dtype, kv_cache=self.cache)
        inv = 1.0 / (v.rope_theta ** (torch.arange(0, v.head_dim, 2, dtype=torch.float32) / v.head_dim))
        ang = torch.arange(self.max_seq, dtype=torch.float32)[:, None] * inv[None]
        self.cos, self.sin = ang.cos().to(dev).contiguous(), ang.sin().to(dev).contiguous()
        self.in_w = g("action_in_proj.weight").to(dev, dtype).contiguous()
        self.in_b = g("action_in_proj.bias").to(dev, dtype).contiguous()
        self._sd_small = {k: sd[k].to(dev, torch.float32) for k in sd
                          if k.startswith(("time_mlp", "action_out_proj")) or ".dense." in k}
        self._schedules: Dict[int, dict] = {}
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        # static denoise-loop state (graph inputs are updated in place)
        i32 = dict(dtype=torch.int32, device=dev)
        Bm, n = max_batch, cfg.horizon
        self.x = torch.zeros(Bm * n, cfg.action_dim, dtype=dtype, device=dev)
        self.h = torch.zeros(Bm * n, e.hidden, dtype=dtype, device=dev)
        self.hn = torch.zeros_like(self.h)
        self.s_pos = torch.zeros(Bm * n, **i32)
        # Every action row is its own one-query "sequence" for the split-KV decode attention kernel: it sees the
        # whole prefix plus all action rows of its sample (their K/V are inserted before attention runs), which
        # is exactly the bidirectional suffix mask, and the KV range is split over many CTAs instead of one.
        self.s_seq = torch.arange(Bm * n, **i32)
        self.s_kvlen = torch.zeros(Bm * n, **i32)
        self.s_pt = torch.zeros((Bm * n, self.cache.pages_per_seq), **i32)
        # the same suffix as one query block per sample (prefill form of the attention launch)
        self.b_qstart = torch.arange(Bm, **i32) * n
        self.b_qlen = torch.full((Bm,), n, **i32)
        self.b_kvlen = torch.zeros(Bm, **i32)
        self.b_seq = torch.arange(Bm, **i32).repeat_interleave(n).contiguous()
        # RF_PI05_SUFFIX_ATTN: `decode` = every suffix row is its own one-token sequence over the sample's pages (split-KV
        # decode kernel: many small CTAs, best at one or two samples); `block` = one bidirectional query block of
        # `horizon` rows per sample (tensor-core prefill kernel: one CTA per sample and head, reads the pages once per
        # sample instead of once per row).  `auto` (default) takes `block` from four samples up: measured denoise loop
        # 14.2 / 51.1 / 97.0 ms (decode) against 20.7 / 45.5 / 58.7 ms (block) at 1 / 8 / 32 samples.
        self.suffix_attn = os.environ.get("RF_PI05_SUFFIX_ATTN", "auto")
        self.prefix_hidden = torch.zeros(Bm * self.max_prefix, v.hidden, dtype=dtype, device=dev)
        # static inputs of the captured prefill: the valid cameras' pixels and the valid language token ids
        S = cfg.vision.image_size
        self.img_in = torch.zeros(Bm * cfg.num_views, 3, S, S, dtype=dtype, device=dev)
        self.ids_in = torch.zeros(Bm * cfg.max_lang_tokens, **i32)
        self._prefill_meta: Dict[tuple, dict] = {}
        self._prefill_graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}

    # ------------------------------------------------------------------ conditioning schedule
    def schedule(self, num_steps: int) -> dict:
        """Per-``num_steps`` constants: adaRMS modulation of every (step, layer, sublayer), the final-norm
        modulation, and the output projection with ``dt`` folded in."""
        hit = self._schedules.get(num_steps)
        if hit is not None:
            return hit
        cfg, sd, e = self.cfg, self._sd_small, self.cfg.expert
        cond = conditioning_schedule(sd, cfg, num_steps)                     # [S, H] fp32 on device
        mods = []
        for i in range(e.layers):
            for n in ("input_layernorm", "post_attention_layernorm"):
                b = f"{EXP}layers.{i}.{n}.dense."
                mods.append(F.linear(cond, sd[b + "weight"], sd[b + "bias"]))
        mod = torch.stack(mods, 1).view(num_steps, e.layers, 2, 1, 3 * e.hidden).to(self.dtype).contiguous()
        fin = F.linear(cond, sd[EXP + "norm.dense.weight"], sd[EXP + "norm.dense.bias"]).to(self.dtype).contiguous()
        dt = -1.0 / num_steps
        hit = dict(mod=mod, final=fin, out_w=(sd["action_out_proj.weight"] * dt).to(self.dtype).contiguous(),
                   out_b=(sd["action_out_proj.bias"] * dt).to(self.dtype).contiguous())
        self._schedules[num_steps] = hit
        return hit

    # ------------------------------------------------------------------ prefix
    def _prefill_geometry(self, im: torch.Tensor, tm: torch.Tensor) -> dict:
        """Device index tensors of one input geometry (which cameras are valid, how many language tokens each sample
        has): built once per geometry, so a repeated geometry copies nothing but pixels and token ids."""
        key = (tuple(im.flatten().tolist()), tuple(tm.sum(1).tolist()))
        hit = self._prefill_meta.get(key)
        if hit is not None:
            return hit
        cfg, dev = self.cfg, self.device
        B = im.shape[0]
        n_img = im.sum(1) * cfg.tokens_per_image
        n_lang = tm.sum(1)
        lens = (n_img + n_lang).to(torch.int32)
        starts = torch.cumsum(lens, 0, dtype=torch.int32) - lens
        lang_rows = torch.cat([torch.arange(int(n_lang[b])) + int(starts[b]) + int(n_img[b]) for b in range(B)])
        img_dst = torch.cat([torch.arange(int(n_img[b])) + int(starts[b]) for b in range(B)])
        pos = torch.cat([torch.arange(int(l), dtype=torch.int32) for l in lens]).to(dev)
        seq = torch.repeat_interleave(torch.arange(B, dtype=torch.int32), lens.long())
        hit = dict(key=key, B=B, T=int(lens.sum()), n_valid=int(im.sum()), n_ids=int(n_lang.sum()), lens=lens.tolist(),
                   longest=int(lens.max()), starts=starts.to(dev), q_len=lens.to(dev), pos=pos, seq=seq.to(dev),
                   lang_rows=lang_rows.to(dev, torch.int32), img_dst=img_dst.to(dev, torch.int32))
        if len(self._prefill_meta) >= 32:
            self._prefill_meta.clear()
            self._prefill_graphs.clear()
        self._prefill_meta[key] = hit
        return hit

    def _prefill_run(self, m: dict) -> None:
        """Vision tower, embedding, packed prefix prefill over the static inputs (device work only)."""
        cfg, K = self.cfg, self.K
        hidden = self.prefix_hidden[:m["T"]]
        if m["n_valid"]:
            img_rows = self.vision(self.img_in[:m["n_valid"]])                         # [n_valid, tok, H]
            K.scatter_rows(hidden, img_rows.reshape(-1, cfg.vlm.hidden), m["img_dst"])
        if m["n_ids"]:
            lang = K.embedding(self.embed, self.ids_in[:m["n_ids"]], scale=math.sqrt(cfg.vlm.hidden))
            K.scatter_rows(hidden, lang, m["lang_rows"])
        self.prefix_stack.forward(hidden, q_start=m["starts"], q_len=m["q_len"], kv_len=m["q_len"], max_q_len=m["longest"],
                                  max_kv_len=m["longest"], pos=m["pos"], cos=self.cos, sin=self.sin, seq_of_tok=m["seq"],
                                  cache_pos=m["pos"], page_table=self.cache.page_table)

    @torch.no_grad()
    def prefill(self, images: torch.Tensor, image_mask: torch.Tensor, tokens: torch.Tensor, token_mask: torch.Tensor, *,
                use_graph: bool = True):
        """Encode the valid cameras and language tokens of every sample and fill the KV cache; returns the per-sample
        prefix lengths (host list).  The device work of one input geometry is captured in a CUDA graph on its first
        use and replayed afterwards; only pixels and token ids are copied per call."""
        B = images.shape[0]
        if B > self.max_batch:
            raise ValueError(f"batch {B} exceeds max_batch {self.max_batch}")
        im = torch.as_tensor(image_mask).bool().cpu()
        tm = torch.as_tensor(token_mask).bool().cpu()
        m = self._prefill_geometry(im, tm)
        if m["n_valid"]:
            flat = images.flatten(0, 1)
            if m["n_valid"] != flat.shape[0]:
                flat = flat[im.flatten().nonzero().flatten().to(flat.device)]
            self.img_in[:m["n_valid"]].copy_(flat, non_blocking=True)
        if m["n_ids"]:
            ids = tokens.cpu()[tm].to(torch.int32)
            self.ids_in[:m["n_ids"]].copy_(ids)
        if not use_graph:
            self._prefill_run(m)
            return m["lens"]
        gph = self._prefill_graphs.get(m["key"])
        if gph is None:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._prefill_run(m)                                     # warm-up: load kernels, fill metadata caches
            torch.cuda.current_stream().wait_stream(s)
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gph, stream=s):
                self._prefill_run(m)
            self._prefill_graphs[m["key"]] = gph
        gph.replay()
        return m["lens"]

    # ------------------------------------------------------------------ denoise
    def _denoise_loop(self, B: int, num_steps: int) -> None:
        cfg, K, sch = self.cfg, self.K, self.schedule(num_steps)
        n, T = cfg.horizon, B * cfg.horizon
        x, h, hn = self.x[:T], self.h[:T], self.hn[:T]
        for s in range(num_steps):
            K.gemm(x, self.in_w, bias=self.in_b, out=h)
            if self.suffix_attn == "block" or (self.suffix_attn == "auto" and B >= 4):
                self.expert_stack.forward(h, q_start=self.b_qstart[:B], q_len=self.b_qlen[:B], kv_len=self.b_kvlen[:B], max_q_len=n,
                                          max_kv_len=self.max_seq, pos=self.s_pos[:T], cos=self.cos, sin=self.sin,
                                          seq_of_tok=self.b_seq[:T], cache_pos=self.s_pos[:T], page_table=self.cache.page_table[:B],
                                          mod=sch["mod"][s], rows_per_mod=T)
            else:
                self.expert_stack.forward(h, decode=True, kv_len=self.s_kvlen[:T], max_kv_len=self.max_seq, pos=self.s_pos[:T],
                                          cos=self.cos, sin=self.sin, seq_of_tok=self.s_seq[:T], cache_pos=self.s_pos[:T],
                                          page_table=self.s_pt[:T], mod=sch["mod"][s], rows_per_mod=T)
            K.rmsnorm(h, None, cfg.expert.eps, out=hn, mod=sch["final"][s:s + 1], rows_per_mod=T)
            K.gemm(hn, sch["out_w"], bias=sch["out_b"], residual=x, out=x)        # x <- x + dt * v

    @torch.no_grad()
    def denoise(self, prefix_lens: Sequence[int], noise: torch.Tensor, num_steps: int = 10, *, use_graph: bool = True):
        cfg, dev = self.cfg, self.device
        B, n = noise.shape[0], cfg.horizon
        T = B * n
        pl = torch.tensor(list(prefix_lens), dtype=torch.int32)
        self.s_kvlen[:T].copy_((pl + n).repeat_interleave(n).to(dev), non_blocking=True)
        self.b_kvlen[:B].copy_((pl + n).to(dev), non_blocking=True)
        self.s_pt[:T].copy_(self.cache.page_table[:B].repeat_interleave(n, 0))
        self.s_pos[:T].copy_((pl[:, None] + torch.arange(n, dtype=torch.int32)[None]).flatten().to(dev), non_blocking=True)
        self.x[:T].copy_(noise.reshape(T, -1).to(dev, self.dtype))
        if not use_graph:
            self._denoise_loop(B, num_steps)
        else:
            key = (B, num_steps)
            gph = self._graphs.get(key)
            if gph is None:
                snap = self.x[:T].clone()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._denoise_loop(B, 1 if num_steps > 1 else num_steps)     # warm-up: load kernels, set attributes
                torch.cuda.current_stream().wait_stream(s)
                self.schedule(num_steps)
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph, stream=s):
                    self._denoise_loop(B, num_steps)
                torch.cuda.synchronize()
                self.x[:T].copy_(snap)
                self._graphs[key] = gph
            gph.replay()
        return self.x[:T].view(B, n, cfg.action_dim)

    @torch.no_grad()
    def predict(self, images, image_mask, tokens, token_mask, noise, num_steps: int = 10, *, use_graph: bool = True):
        lens = self.prefill(images, image_mask, tokens, token_mask, use_graph=use_graph)
        return self.denoise(lens, noise, num_steps, use_graph=use_graph)

    def check_status(self) -> None:
        self.prefix_stack.check_status()
        self.expert_stack.check_status()
        self.vision.tower.stack.check_status()

    def close(self) -> None:
        self._graphs.clear()
        self._prefill_graphs.clear()
        self.vision.close()
        self.prefix_stack.close()
        self.expert_stack.close()
        self.cache.close()
