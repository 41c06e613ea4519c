"""Wall-OSS: a Qwen2.5-VL prefix ("expert 0") and a narrow dense flow-matching action decoder ("expert 1") that
share one KV cache.

Every decoder layer of the checkpoint holds two sets of weights: expert 0 (width 2048, MLP 11008) reads the
multimodal prompt, expert 1 (width 1024, MLP 2048) reads the noisy action chunk.  Both project to the same attention
geometry (16 query heads, 2 KV heads of 128), so the action rows attend to the prompt's keys and values directly.

Data flow of one action chunk:

  camera images + prompt tokens -> Qwen2.5-VL (windowed vision tower, chunked M-RoPE decoder), one packed prefill:
  K/V of every layer land in the paged cache at rows [0, P)
  x_0 = noise [horizon, action_dim]; times = linspace(0, 1, num_steps + 1), dt = 1 / num_steps; for step k:
      e = w3( silu( w2( [ w1([x | dof_mask]) | sincos(t_k) ] ) ) )                      (horizon rows of width 1024)
      expert-1 layer i: RMSNorm -> q/k/v (+bias) -> RoPE at p0 + row (p0 = largest prompt position + 1, the same
          value on the three M-RoPE axes) -> K/V written at cache rows P + row -> attention over
          [prompt rows | action rows] under the action mask -> o_proj -> residual; RMSNorm -> SwiGLU MLP -> residual
      v = action_proj_back(rmsnorm(h));  v <- v * dof_mask + (padding - noise) * (1 - dof_mask);  x <- x + dt * v

Action mask: every action row sees the whole prompt; among themselves the rows are causal (stock checkpoints) or
bidirectional (checkpoints trained that way).

What only depends on the step index is computed once per ``num_steps``: ``w2[:, :AH] @ w1`` collapses the two input
projections into one GEMM whose K dimension carries ``[x | dof_mask]``, the time half of ``w2`` becomes a per-step
bias, and ``dt`` is folded into ``action_proj_back`` so that the Euler update is that GEMM's residual epilogue.  The
loop replays from one CUDA graph; prompt length, positions, mask and page table live in device buffers at fixed
addresses.

Reference behaviour: ``python/rpu_backend/adapters/wall_oss/action.py:52-58,66-112,408-418,495-553,1033-1165,1251-1284``
(time embedding, masked-DOF blend, preprocessor, mask, schedule, expert-1 tensor names, weight folding),
``adapters/wall_oss/llm.py:1-30,1060-1245`` (expert-0 names), ``adapters/wall_oss/runtime.py:1247-1420`` (orchestration),
``src/fused/rpu_wall_oss_action_step_model.h:1-18`` (fused step).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, Iterator, List, Optional, Tuple

import torch
import torch.nn.functional as F

from .decoder import DecoderConfig
from .qwen25_vl_vision import Qwen25VLVisionConfig

PRE_P = "action_preprocessor."


@dataclass
class WallOssConfig:
    hidden: int = 1024            # width of expert 1 (and of the action preprocessor)
    inter: int = 2048
    layers: int = 36
    heads: int = 16
    kv_heads: int = 2
    head_dim: int = 128
    eps: float = 1e-6
    rope_theta: float = 1e6
    action_dim: int = 26
    horizon: int = 32
    num_steps: int = 10
    causal_actions: bool = True
    flow_time_scale: float = 1.0


def tiny_wall_oss_config(**kw) -> WallOssConfig:
    base = dict(hidden=64, inter=128, layers=3, heads=2, kv_heads=1, head_dim=64, rope_theta=1e4, action_dim=6, horizon=8,
                num_steps=4)
    base.update(kw)
    return WallOssConfig(**base)


# ----------------------------------------------------------------------------- checkpoint names
def wall_oss_expert_shapes(cfg: WallOssConfig, expert: int = 1, *, hidden: Optional[int] = None,
                           inter: Optional[int] = None) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """(checkpoint name, shape, kind) of the decoder tensors of one expert (fused QKV and gate/up, per-expert norms)."""
    H, I = hidden or cfg.hidden, inter or cfg.inter
    qkv = (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim
    for i in range(cfg.layers):
        b = f"model.layers.{i}."
        yield b + f"self_attn.qkv_proj_experts.{expert}.weight", (qkv, H), "matrix"
        yield b + f"self_attn.qkv_proj_experts.{expert}.bias", (qkv,), "bias"
        yield b + f"self_attn.o_proj_experts.{expert}.weight", (H, cfg.heads * cfg.head_dim), "matrix"
        yield b + f"moe.experts.{expert}.gate_up_proj.weight", (2 * I, H), "matrix"
        yield b + f"moe.experts.{expert}.down_proj.weight", (H, I), "matrix"
        yield b + f"input_layernorms.{expert}.weight", (H,), "norm"
        yield b + f"post_attention_layernorms.{expert}.weight", (H,), "norm"
    yield f"model.norms.{expert}.weight", (H,), "norm"


def wall_oss_action_shapes(cfg: WallOssConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    AH, AD = cfg.hidden, cfg.action_dim
    yield PRE_P + "w1.weight", (AH, 2 * AD), "matrix"
    yield PRE_P + "w2.weight", (AH, 2 * AH), "matrix"
    yield PRE_P + "w3.weight", (AH, AH), "matrix"
    yield PRE_P + "action_proj_back.weight", (AD, AH), "matrix"


def random_wall_oss_expert(cfg: WallOssConfig, *, seed: int = 0, std: float = 0.05, dtype=torch.float16,
                           device="cpu") -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in list(wall_oss_expert_shapes(cfg)) + list(wall_oss_action_shapes(cfg)):
        r = torch.randn(shape, generator=g)
        sd[name] = {"matrix": r * std, "norm": 1.0 + 0.05 * r, "bias": 0.03 * r}[kind].to(device, dtype)
    return sd


def expert0_getter(get_weight: Callable[[str], torch.Tensor], text: DecoderConfig, names=None) -> Callable[[str], torch.Tensor]:
    """Serve expert 0 under plain causal-LM names (``model.layers.N.self_attn.q_proj.weight`` ...) out of the fused
    per-expert tensors.  The last fused tensor read is kept, so q, k and v (or gate and up) cost one read."""
    hd, nq, nkv, I = text.head_dim, text.num_heads, text.num_kv_heads, text.intermediate_size
    rows = {"q": (0, nq * hd), "k": (nq * hd, (nq + nkv) * hd), "v": ((nq + nkv) * hd, (nq + 2 * nkv) * hd)}
    last: List = [None, None]

    def fused(name: str) -> torch.Tensor:
        if last[0] != name:
            last[0], last[1] = name, get_weight(name)
        return last[1]

    def get(name: str) -> torch.Tensor:
        if name == "model.norm.weight":
            return get_weight("model.norms.0.weight")
        if name == "lm_head.weight":
            if names is not None and "lm_head.weight" not in names:
                return get_weight("model.embed_tokens.weight")
            return get_weight(name)
        if not name.startswith("model.layers."):
            return get_weight(name)
        _, _, idx, rest = name.split(".", 3)
        b = f"model.layers.{idx}."
        if rest.startswith("self_attn.") and rest[10] in "qkv" and rest[11:17] == "_proj.":
            lo, hi = rows[rest[10]]
            return fused(b + "self_attn.qkv_proj_experts.0." + rest[17:])[lo:hi]
        if rest == "self_attn.o_proj.weight":
            return get_weight(b + "self_attn.o_proj_experts.0.weight")
        if rest in ("mlp.gate_proj.weight", "mlp.up_proj.weight"):
            gu = fused(b + "moe.experts.0.gate_up_proj.weight")
            half = gu.shape[0] // 2
            return gu[:I] if rest.startswith("mlp.gate") else gu[half:half + I]
        if rest == "mlp.down_proj.weight":
            return get_weight(b + "moe.experts.0.down_proj.weight")[:, :I]
        if rest == "input_layernorm.weight":
            return get_weight(b + "input_layernorms.0.weight")
        if rest == "post_attention_layernorm.weight":
            return get_weight(b + "post_attention_layernorms.0.weight")
        raise KeyError(name)
    return get


class VisionNames(dict):
    """The vision tower's tensors under ``blocks.N.mlp.{gate,up}_proj.*`` out of the checkpoint's fused
    ``visual.blocks.N.mlp.gate_up_proj.*`` (two equal halves, each possibly zero-padded past the logical width)."""

    def __init__(self, get_weight: Callable[[str], torch.Tensor], inter: int, prefix: str = "visual."):
        super().__init__()
        self._get, self._inter, self._prefix = get_weight, inter, prefix

    def __missing__(self, key: str) -> torch.Tensor:
        for part, first in (("mlp.gate_proj.", True), ("mlp.up_proj.", False)):
            if part in key:
                t = self._get(self._prefix + key.replace(part, "mlp.gate_up_proj."))
                half = t.shape[0] // 2
                return t[:self._inter] if first else t[half:half + self._inter]
        t = self._get(self._prefix + key)
        if key.endswith("mlp.down_proj.weight"):
            t = t[:, :self._inter]
        return t


# ----------------------------------------------------------------------------- schedule pieces
def sinusoidal_pos_emb(t: torch.Tensor, dim: int) -> torch.Tensor:
    """``[n] -> [n, dim]`` fp32: sin | cos over ``dim / 2`` frequencies ``10000^(-i / (dim/2 - 1))``."""
    half = dim // 2
    freq = torch.exp(torch.arange(half, dtype=torch.float32) * -(math.log(10000.0) / (half - 1)))
    ang = t.float()[:, None] * freq[None, :]
    return torch.cat((ang.sin(), ang.cos()), -1)


def flow_times(num_steps: int, scale: float = 1.0) -> torch.Tensor:
    t = torch.linspace(0, 1, num_steps + 1)
    return t if scale == 1.0 else t * scale


def action_mask(prefix_len: int, horizon: int, width: int, *, causal: bool = True) -> torch.Tensor:
    """Boolean ``[horizon, width]``: cache rows each action row attends to (prompt rows, then the action rows)."""
    m = torch.zeros(horizon, width, dtype=torch.bool)
    m[:, :prefix_len] = True
    blk = torch.ones(horizon, horizon, dtype=torch.bool)
    m[:, prefix_len:prefix_len + horizon] = torch.tril(blk) if causal else blk
    return m


def masked_dof_inputs(noise: torch.Tensor, dof_mask: torch.Tensor, padding_action: Optional[torch.Tensor]):
    """``(mask, override)`` of the velocity blend ``v * mask + override`` with ``override = (padding - noise) * (1 - mask)``,
    or ``(None, None)`` when every degree of freedom is active.  Inactive dimensions then travel on a straight line from
    their noise value to ``padding_action`` (normalised physical zero) over the unit time interval."""
    if tuple(dof_mask.shape) != tuple(noise.shape):
        raise ValueError(f"dof_mask must match noise shape {tuple(noise.shape)}, got {tuple(dof_mask.shape)}")
    mask = dof_mask.detach().to("cpu", torch.float32).contiguous()
    if not bool(((mask == 0) | (mask == 1)).all()):
        raise ValueError("dof_mask must contain only 0 or 1")
    if bool((mask == 1).all()):
        return None, None
    if padding_action is None:
        raise ValueError("padding_action is required when dof_mask contains inactive dimensions")
    if tuple(padding_action.shape) != tuple(noise.shape):
        raise ValueError(f"padding_action must match noise shape {tuple(noise.shape)}, got {tuple(padding_action.shape)}")
    pad = padding_action.detach().to("cpu", torch.float32)
    if not bool(torch.isfinite(pad).all()):
        raise ValueError("padding_action must contain only finite values")
    return mask, ((pad - noise.detach().to("cpu", torch.float32)) * (1.0 - mask)).contiguous()


def folded_preprocessor(sd: Dict[str, torch.Tensor], cfg: WallOssConfig, num_steps: int):
    """``(W [AH, 2 * action_dim], step_bias [num_steps, AH])`` fp32 with
    ``silu([x | dof] @ W.T + step_bias[k]) == silu(w2(cat(w1([x | dof]), sincos(t_k))))``."""
    AH = cfg.hidden
    w1, w2 = sd[PRE_P + "w1.weight"].float(), sd[PRE_P + "w2.weight"].float()
    te = sinusoidal_pos_emb(flow_times(num_steps, cfg.flow_time_scale)[:-1], AH).to(w2.device)
    return (w2[:, :AH] @ w1).contiguous(), (te @ w2[:, AH:].t()).contiguous()


# ----------------------------------------------------------------------------- fp32 oracle of expert 1
class TorchWallOssExpert:
    """Plain PyTorch statement of the denoise loop over given prompt K/V (``[layers] x (K, V)`` of shape
    ``[kv_heads, P, head_dim]``, already rotated), with none of the engine's folds."""

    def __init__(self, cfg: WallOssConfig, sd: Dict[str, torch.Tensor], *, dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.sd = {k: v.to(self.device, dtype) for k, v in sd.items()}

    def _rope(self, t, pos):      # t [heads, n, hd]
        cfg = self.cfg
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32, device=self.device) / cfg.head_dim))
        ang = pos.float()[None, :, None] * inv
        cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)
        h = t.shape[-1] // 2
        return (t.float() * cos + torch.cat((-t[..., h:], t[..., :h]), -1).float() * sin).to(t.dtype)

    @torch.no_grad()
    def sample_actions(self, prefix_kv, prefix_len: int, p0: int, noise: torch.Tensor, dof_mask: torch.Tensor,
                       num_steps: Optional[int] = None, padding_action: Optional[torch.Tensor] = None) -> torch.Tensor:
        cfg, sd = self.cfg, self.sd
        num_steps = num_steps or cfg.num_steps
        n, AH, hd, I = cfg.horizon, cfg.hidden, cfg.head_dim, cfg.inter
        G = cfg.heads // cfg.kv_heads
        nq, nkv = cfg.heads * hd, cfg.kv_heads * hd
        x = noise.reshape(n, cfg.action_dim).to(self.device, self.dtype)
        dof = dof_mask.reshape(n, cfg.action_dim).to(self.device, self.dtype)
        bm, ovr = masked_dof_inputs(noise.reshape(n, -1), dof_mask.reshape(n, -1),
                                    None if padding_action is None else padding_action.reshape(n, -1))
        times = flow_times(num_steps, cfg.flow_time_scale)
        dt = float(times[1] - times[0])
        mask = action_mask(prefix_len, n, prefix_len + n, causal=cfg.causal_actions).to(self.device)
        pos = p0 + torch.arange(n, device=self.device)

        def rms(t, w):
            tf = t.float()
            return (tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + cfg.eps) * w.float()).to(self.dtype)
        for k in range(num_steps):
            te = sinusoidal_pos_emb(times[k:k + 1], AH).to(self.device, self.dtype).expand(n, -1)
            ae = F.linear(torch.cat((x, dof), -1), sd[PRE_P + "w1.weight"])
            h = F.linear(F.silu(F.linear(torch.cat((ae, te), -1), sd[PRE_P + "w2.weight"])), sd[PRE_P + "w3.weight"])
            for i in range(cfg.layers):
                b = f"model.layers.{i}."
                y = rms(h, sd[b + "input_layernorms.1.weight"])
                qkv = F.linear(y, sd[b + "self_attn.qkv_proj_experts.1.weight"], sd[b + "self_attn.qkv_proj_experts.1.bias"])
                q = qkv[:, :nq].view(n, cfg.heads, hd).transpose(0, 1)
                kk = qkv[:, nq:nq + nkv].view(n, cfg.kv_heads, hd).transpose(0, 1)
                vv = qkv[:, nq + nkv:].view(n, cfg.kv_heads, hd).transpose(0, 1)
                q, kk = self._rope(q, pos), self._rope(kk, pos)
                ka = torch.cat((prefix_kv[i][0].to(self.device, self.dtype), kk), 1).repeat_interleave(G, 0)
                va = torch.cat((prefix_kv[i][1].to(self.device, self.dtype), vv), 1).repeat_interleave(G, 0)
                s = (q.float() @ ka.float().transpose(-1, -2)) / math.sqrt(hd)
                s = s.masked_fill(~mask[None], float("-inf"))
                o = (torch.softmax(s, -1) @ va.float()).to(self.dtype).transpose(0, 1).reshape(n, -1)
                h = h + F.linear(o, sd[b + "self_attn.o_proj_experts.1.weight"])
                y = rms(h, sd[b + "post_attention_layernorms.1.weight"])
                gu = F.linear(y, sd[b + "moe.experts.1.gate_up_proj.weight"])
                h = h + F.linear(F.silu(gu[:, :I]) * gu[:, I:2 * I], sd[b + "moe.experts.1.down_proj.weight"])
            v = F.linear(rms(h, sd["model.norms.1.weight"]), sd[PRE_P + "action_proj_back.weight"])
            if bm is not None:
                v = v * bm.to(self.device, self.dtype) + ovr.to(self.device, self.dtype)
            x = x + dt * v
        return x


# ----------------------------------------------------------------------------- device engine
class WallOssEngine:
    """Qwen2.5-VL prompt decoder + dense action decoder on the accelerator.  ``predict(...)`` returns the normalised
    ``[horizon, action_dim]`` chunk in a stable buffer that the next call overwrites."""

    def __init__(self, cfg: WallOssConfig, text: DecoderConfig, vcfg: Qwen25VLVisionConfig,
                 get_weight: Callable[[str], torch.Tensor], *, names: Optional[set] = None, image_token_id: int = 151655,
                 device="cuda", dtype=torch.float16, max_prefix: int = 1024, max_patches: int = 4096):
        from ..ops import kernels as K
        from ..runtime.stack import NativeStack, StackSpec
        from .qwen25_vl import Qwen25VLEngine
        self.K, self.cfg, self.device, self.dtype = K, cfg, torch.device(device), dtype
        dev = self.device
        n = cfg.horizon
        if (text.num_layers, text.num_heads, text.num_kv_heads, text.head_dim) != (cfg.layers, cfg.heads, cfg.kv_heads, cfg.head_dim):
            raise ValueError("the two experts must share the attention geometry (layers, heads, kv heads, head_dim): "
                             f"{(text.num_layers, text.num_heads, text.num_kv_heads, text.head_dim)} vs "
                             f"{(cfg.layers, cfg.heads, cfg.kv_heads, cfg.head_dim)}")
        self.max_prefix = max_prefix
        self.max_seq = (max_prefix + n + 15) // 16 * 16
        self.vlm = Qwen25VLEngine(text, vcfg, expert0_getter(get_weight, text, names),
                                  VisionNames(get_weight, vcfg.intermediate_size), image_token_id=image_token_id,
                                  device=device, dtype=dtype, max_seq_len=self.max_seq, max_patches=max_patches,
                                  max_prefill_tokens=max(max_prefix, 256))
        self.cache = self.vlm.text.cache
        self.image_token_id = image_token_id
        g = get_weight
        I = cfg.inter
        layers = []
        for i in range(cfg.layers):
            b = f"model.layers.{i}."
            gu = g(b + "moe.experts.1.gate_up_proj.weight")
            half = gu.shape[0] // 2
            layers.append(dict(
                norm1_w=g(b + "input_layernorms.1.weight"), norm2_w=g(b + "post_attention_layernorms.1.weight"),
                wqkv=g(b + "self_attn.qkv_proj_experts.1.weight"), bqkv=g(b + "self_attn.qkv_proj_experts.1.bias"),
                wo=g(b + "self_attn.o_proj_experts.1.weight"), w_up=torch.cat((gu[:I], gu[half:half + I]), 0),
                w_down=g(b + "moe.experts.1.down_proj.weight")[:, :I]))
        self.rows = (n + 15) // 16 * 16
        self.expert = NativeStack(
            StackSpec(layers=cfg.layers, hidden=cfg.hidden, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
                      inter=I, norm="rms", mlp="swiglu", eps=cfg.eps, rot_dim=cfg.head_dim, paged_kv=True, causal=False,
                      max_tokens=self.rows, max_seqs=1),
            layers, device=device, dtype=dtype, kv_cache=self.cache)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32) / cfg.head_dim))
        ang = torch.arange(self.max_seq + 4096, dtype=torch.float32)[:, None] * inv[None]
        self.cos, self.sin = ang.cos().to(dev).contiguous(), ang.sin().to(dev).contiguous()
        self._small = {k: g(k).to(dev, torch.float32) for k, _, _ in wall_oss_action_shapes(cfg)}
        self.final_norm_w = g("model.norms.1.weight").to(dev, dtype).contiguous()
        self.k_pad = (2 * cfg.action_dim + 7) // 8 * 8          # GEMM K and N are multiples of 8
        self._schedules: Dict[int, dict] = {}
        self._graphs: Dict[Tuple[int, bool], torch.cuda.CUDAGraph] = {}
        i32 = dict(dtype=torch.int32, device=dev)
        AH = cfg.hidden
        self.x = torch.zeros(n, self.k_pad, dtype=dtype, device=dev)        # [x | dof_mask | 0]
        self.v = torch.zeros(n, self.k_pad, dtype=dtype, device=dev)
        self.blend = torch.zeros(n, self.k_pad, dtype=dtype, device=dev)    # dof mask over the x columns, 0 elsewhere
        self.ovr = torch.zeros(n, self.k_pad, dtype=dtype, device=dev)      # dt * (padding - noise) * (1 - mask)
        self.h = torch.zeros(n, AH, dtype=dtype, device=dev)
        self.hn = torch.zeros(n, AH, dtype=dtype, device=dev)
        self.enc = torch.zeros(n, AH, dtype=dtype, device=dev)
        self.s_pos = torch.zeros(n, **i32)
        self.s_cache_pos = torch.zeros(n, **i32)
        self.s_seq = torch.zeros(n, **i32)
        self.s_qstart = torch.zeros(1, **i32)
        self.s_qlen = torch.full((1,), n, **i32)
        self.s_kvlen = torch.zeros(1, **i32)
        self.mask = torch.zeros(n, (self.max_seq + 127) // 128 * 128, dtype=torch.uint8, device=dev)[:, :self.max_seq]   # pitch: whole 128-key blocks

    # ------------------------------------------------------------------ per-num_steps constants
    def schedule(self, num_steps: int) -> dict:
        hit = self._schedules.get(num_steps)
        if hit is not None:
            return hit
        cfg, sd = self.cfg, self._small
        w, sb = folded_preprocessor(sd, cfg, num_steps)
        times = flow_times(num_steps, cfg.flow_time_scale)
        dt = float(times[1] - times[0])
        pad = lambda m, rows, cols: F.pad(m, (0, cols - m.shape[1], 0, rows - m.shape[0]))
        hit = dict(dt=dt,
                   enc_w=pad(w, cfg.hidden, self.k_pad).to(self.dtype).contiguous(),
                   enc_b=sb.to(self.dtype).contiguous(),
                   w3=sd[PRE_P + "w3.weight"].to(self.dtype).contiguous(),
                   out_w=pad(sd[PRE_P + "action_proj_back.weight"] * dt, self.k_pad, cfg.hidden).to(self.dtype).contiguous())
        self._schedules[num_steps] = hit
        return hit

    # ------------------------------------------------------------------ prompt
    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor], image_grid_thw) -> Tuple[int, int]:
        """Fill the KV cache with the prompt; returns ``(prompt rows P, first action rope position p0)``."""
        P = int(input_ids.numel())
        if P > self.max_prefix:
            raise ValueError(f"prompt of {P} rows exceeds max_prefix {self.max_prefix}")
        self.vlm.prefill(input_ids, pixel_values, image_grid_thw)
        return P, int(self.vlm._next_pos)

    # ------------------------------------------------------------------ denoise
    def _denoise_loop(self, num_steps: int, blend: bool) -> None:
        cfg, K, sch = self.cfg, self.K, self.schedule(num_steps)
        n = cfg.horizon
        for k in range(num_steps):
            K.gemm(self.x, sch["enc_w"], bias=sch["enc_b"][k], act="silu", out=self.enc)
            K.gemm(self.enc, sch["w3"], out=self.h)
            self.expert.forward(self.h, q_start=self.s_qstart, q_len=self.s_qlen, kv_len=self.s_kvlen, max_q_len=n,
                                max_kv_len=self.max_seq, pos=self.s_pos, cos=self.cos, sin=self.sin,
                                seq_of_tok=self.s_seq, cache_pos=self.s_cache_pos, page_table=self.cache.page_table,
                                mask=self.mask)
            K.rmsnorm(self.h, self.final_norm_w, cfg.eps, out=self.hn)
            if not blend:
                K.gemm(self.hn, sch["out_w"], residual=self.x, out=self.x)      # x <- x + dt * v (dof columns: + 0)
            else:
                K.gemm(self.hn, sch["out_w"], out=self.v)
                self.x.addcmul_(self.v, self.blend).add_(self.ovr)

    @torch.no_grad()
    def denoise(self, prefix_len: int, p0: int, noise: torch.Tensor, dof_mask: Optional[torch.Tensor] = None,
                num_steps: Optional[int] = None, *, padding_action: Optional[torch.Tensor] = None,
                use_graph: bool = True) -> torch.Tensor:
        cfg, dev = self.cfg, self.device
        num_steps = num_steps or cfg.num_steps
        n, AD = cfg.horizon, cfg.action_dim
        noise = noise.reshape(n, AD).to("cpu", torch.float32)
        dof = torch.ones(n, AD) if dof_mask is None else dof_mask.reshape(n, AD).to("cpu", torch.float32)
        bm, ovr = masked_dof_inputs(noise, dof, None if padding_action is None else padding_action.reshape(n, AD))
        blend = bm is not None
        sch = self.schedule(num_steps)
        self.cache.ensure(0, prefix_len + n)
        self.cache.sync_table()
        ar = torch.arange(n, dtype=torch.int32)
        self.s_pos.copy_((ar + p0).to(dev), non_blocking=True)
        self.s_cache_pos.copy_((ar + prefix_len).to(dev), non_blocking=True)
        self.s_kvlen.fill_(prefix_len + n)
        self.mask.copy_(action_mask(prefix_len, n, self.max_seq, causal=cfg.causal_actions).to(torch.uint8).to(dev),
                        non_blocking=True)
        x0 = torch.zeros(n, self.k_pad)
        x0[:, :AD], x0[:, AD:2 * AD] = noise, dof
        self.x.copy_(x0.to(dev, self.dtype))
        if blend:
            b0, o0 = torch.zeros(n, self.k_pad), torch.zeros(n, self.k_pad)
            b0[:, :AD], o0[:, :AD] = bm, ovr * sch["dt"]
            self.blend.copy_(b0.to(dev, self.dtype))
            self.ovr.copy_(o0.to(dev, self.dtype))
        if not use_graph:
            self._denoise_loop(num_steps, blend)
        else:
            gph = self._graphs.get((num_steps, blend))
            if gph is None:
                snap = self.x.clone()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._denoise_loop(1, blend)                     # warm-up: load kernels, set attributes
                torch.cuda.current_stream().wait_stream(s)
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph, stream=s):
                    self._denoise_loop(num_steps, blend)
                torch.cuda.synchronize()
                self.x.copy_(snap)
                self._graphs[(num_steps, blend)] = gph
            gph.replay()
        return self.x[:, :AD]

    @torch.no_grad()
    def predict(self, input_ids, pixel_values, image_grid_thw, noise, dof_mask=None, num_steps: Optional[int] = None, *,
                padding_action=None, use_graph: bool = True) -> torch.Tensor:
        P, p0 = self.prefill(input_ids, pixel_values, image_grid_thw)
        return self.denoise(P, p0, noise, dof_mask, num_steps, padding_action=padding_action, use_graph=use_graph)

    def check_status(self) -> None:
        self.vlm.text.check_status()
        self.expert.check_status()

    def close(self) -> None:
        self._graphs.clear()
        self.expert.close()
        self.vlm.close()


__all__ = ["WallOssConfig", "WallOssEngine", "TorchWallOssExpert", "tiny_wall_oss_config", "wall_oss_expert_shapes",
           "wall_oss_action_shapes", "random_wall_oss_expert", "expert0_getter", "VisionNames", "sinusoidal_pos_emb",
           "flow_times", "action_mask", "masked_dof_inputs", "folded_preprocessor"]
