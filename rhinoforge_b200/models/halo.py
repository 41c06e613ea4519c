"""HALO: a Qwen2.5-with-QK-norm decoder as a mixture of transformers, run as an action expert and as an image-flow step.

Every decoder layer holds the text ("understanding") weights and twin sets with a module-name suffix: ``_moe_act`` for
action rows, ``_moe_gen`` for VAE-latent rows.  Norms, q/k/v (with bias) / o, the per-head q/k norms and the MLP all come
in pairs, and so does the final norm.  A query chunk mixes rows of both kinds (action mode: text rows 0 and 17 around 16
action rows; generation mode: start / end-of-image text rows around 1376 latent rows); each row runs through the set
of its kind, attention then mixes all rows with the prefix's keys and values (full, non-causal attention: every row sees
the whole prefix and the whole chunk), and all rows of a chunk share ONE rotary position.

One denoise step is: compose the chunk's input rows (action mode: ``input_linear(x_t) + time_mlp(t) + sinusoidal
position``; generation mode: ``vae2llm(x_t) + time_mlp(t) + latent position table``; text rows from the embedding table),
run the twin-weight decoder over the prefix cache, final norm per kind, project the non-text rows back
(``output_linear`` / ``llm2vae``) and take a backward Euler step ``x <- x - v * dt`` along ``linspace(1, 0, n)``.

Here the chunk's rows are ordered ``[text rows | twin rows]`` (the native stack routes by row range; cache rows keep the
chunk's own order), everything that depends on the step index only is a per-step bias, ``-dt`` is folded into the
output projection so the Euler update is that GEMM's residual epilogue, and the action loop replays from one CUDA graph.

Reference behaviour: ``src/fused/rpu_halo_action_expert_model.h:1-60``, ``src/fused/rpu_halo_image_flow_model.h:1-40``
(twin weights, row-mask merge, chunk layouts), ``python/rpu_backend/adapters/halo/weights.py:1-30,160-190,299-322`` (names,
embeddings), ``adapters/halo/runtime.py:81-96,255-283,325-366`` (schedule, input rows, rollout).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

LAYERS_P = "language_model.model.layers."
MODEL_P = "language_model.model."
SUFFIX = {"act": "_moe_act", "gen": "_moe_gen"}


@dataclass
class HaloConfig:
    layers: int = 28
    hidden: int = 1536
    heads: int = 12
    kv_heads: int = 2
    head_dim: int = 128
    inter: int = 8960
    eps: float = 1e-6
    rope_theta: float = 1e6
    vocab: int = 151933
    action_rows: int = 16            # action mode: chunk = text row, action rows, text row
    action_dim: int = 14
    time_freq_dim: int = 256
    time_max_period: float = 1e4
    latent_dim: int = 64             # generation mode: VAE latent width
    latent_rows: int = 1376
    max_latent_size: int = 32        # side of the latent position table

    def chunk_rows(self, mode: str) -> int:
        return 2 + (self.action_rows if mode == "act" else self.latent_rows)


def tiny_halo_config(**kw) -> HaloConfig:
    base = dict(layers=3, hidden=128, heads=2, kv_heads=1, head_dim=64, inter=256, rope_theta=1e4, vocab=40, action_rows=6,
                action_dim=5, time_freq_dim=32, latent_dim=16, latent_rows=20, max_latent_size=6)
    base.update(kw)
    return HaloConfig(**base)


def halo_shapes(cfg: HaloConfig, mode: str = "act") -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """(checkpoint name, shape, kind) of the text set, the twin set of ``mode`` and that mode's head."""
    H, hd, I = cfg.hidden, cfg.head_dim, cfg.inter
    for i in range(cfg.layers):
        b = f"{LAYERS_P}{i}."
        for s in ("", SUFFIX[mode]):
            for n, rows in (("q", cfg.heads), ("k", cfg.kv_heads), ("v", cfg.kv_heads)):
                yield b + f"self_attn.{n}_proj{s}.weight", (rows * hd, H), "matrix"
                yield b + f"self_attn.{n}_proj{s}.bias", (rows * hd,), "bias"
            yield b + f"self_attn.o_proj{s}.weight", (H, cfg.heads * hd), "matrix"
            yield b + f"self_attn.q_norm{s}.weight", (hd,), "norm"
            yield b + f"self_attn.k_norm{s}.weight", (hd,), "norm"
            yield b + f"input_layernorm{s}.weight", (H,), "norm"
            yield b + f"post_attention_layernorm{s}.weight", (H,), "norm"
            yield b + f"mlp{s}.gate_proj.weight", (I, H), "matrix"
            yield b + f"mlp{s}.up_proj.weight", (I, H), "matrix"
            yield b + f"mlp{s}.down_proj.weight", (H, I), "matrix"
    yield MODEL_P + "norm.weight", (H,), "norm"
    yield MODEL_P + f"norm{SUFFIX[mode]}.weight", (H,), "norm"
    yield MODEL_P + "embed_tokens.weight", (cfg.vocab, H), "embed"
    t = "action_time_embedder" if mode == "act" else "time_embedder"
    yield t + ".mlp.0.weight", (H, cfg.time_freq_dim), "matrix"
    yield t + ".mlp.0.bias", (H,), "bias"
    yield t + ".mlp.2.weight", (H, H), "matrix"
    yield t + ".mlp.2.bias", (H,), "bias"
    if mode == "act":
        yield "input_linear_layer.weight", (H, cfg.action_dim), "matrix"
        yield "input_linear_layer.bias", (H,), "bias"
        yield "output_linear_layer.weight", (cfg.action_dim, H), "matrix"
        yield "output_linear_layer.bias", (cfg.action_dim,), "bias"
    else:
        yield "vae2llm.weight", (H, cfg.latent_dim), "matrix"
        yield "vae2llm.bias", (H,), "bias"
        yield "llm2vae.weight", (cfg.latent_dim, H), "matrix"
        yield "llm2vae.bias", (cfg.latent_dim,), "bias"
        yield "latent_pos_embed.pos_embed", (cfg.max_latent_size ** 2, H), "embed"


def random_halo_state_dict(cfg: HaloConfig, mode: str = "act", *, seed: int = 0, std: float = 0.06,
                           dtype=torch.float32) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in halo_shapes(cfg, mode):
        r = torch.randn(shape, generator=g)
        sd[name] = {"matrix": r * std, "embed": r * 0.3, "norm": 1.0 + 0.05 * r, "bias": 0.03 * r}[kind].to(dtype)
    return sd


# ----------------------------------------------------------------------------- embeddings and schedule
def timestep_embedding(t: torch.Tensor, cfg: HaloConfig) -> torch.Tensor:
    """``[n] -> [n, time_freq_dim]`` fp32: cos | sin over ``max_period^(-i / half)``."""
    half = cfg.time_freq_dim // 2
    freqs = torch.exp(-math.log(cfg.time_max_period) * torch.arange(half, dtype=torch.float32) / half)
    args = t.float()[:, None] * freqs[None, :]
    return torch.cat((args.cos(), args.sin()), -1)


def sinusoidal_pos_embedding(position_ids: torch.Tensor, cfg: HaloConfig) -> torch.Tensor:
    """``[n] -> [n, hidden]`` fp32: sin | cos over ``max_period^(-i / (half - 1))``."""
    half = cfg.hidden // 2
    freqs = torch.exp(torch.arange(half, dtype=torch.float32) * -(math.log(cfg.time_max_period) / (half - 1)))
    args = position_ids.float()[:, None] * freqs[None, :]
    return torch.cat((args.sin(), args.cos()), -1)


def euler_schedule(num_timesteps: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(t_i, dt_i)`` of the fixed backward Euler loop: ``t = linspace(1, 0, n)``, ``n - 1`` steps, ``x <- x - v * dt``."""
    if num_timesteps < 2:
        raise ValueError(f"num_timesteps must be >= 2, got {num_timesteps}")
    t = torch.linspace(1, 0, num_timesteps)
    return t[:-1], t[:-1] - t[1:]


def _time_mlp(sd, cfg: HaloConfig, mode: str, t: torch.Tensor) -> torch.Tensor:
    p = "action_time_embedder" if mode == "act" else "time_embedder"
    f = timestep_embedding(t.cpu(), cfg).to(sd[p + ".mlp.0.weight"].device)
    return F.linear(F.silu(F.linear(f, sd[p + ".mlp.0.weight"].float(), sd[p + ".mlp.0.bias"].float())),
                    sd[p + ".mlp.2.weight"].float(), sd[p + ".mlp.2.bias"].float())


def _branch_layers(sd, cfg: HaloConfig, s: str) -> List[Dict[str, torch.Tensor]]:
    out = []
    for i in range(cfg.layers):
        b = f"{LAYERS_P}{i}."
        out.append(dict(
            norm1_w=sd[b + f"input_layernorm{s}.weight"], norm2_w=sd[b + f"post_attention_layernorm{s}.weight"],
            wqkv=torch.cat([sd[b + f"self_attn.{x}_proj{s}.weight"] for x in "qkv"], 0),
            bqkv=torch.cat([sd[b + f"self_attn.{x}_proj{s}.bias"] for x in "qkv"], 0),
            wo=sd[b + f"self_attn.o_proj{s}.weight"], q_norm_w=sd[b + f"self_attn.q_norm{s}.weight"],
            k_norm_w=sd[b + f"self_attn.k_norm{s}.weight"],
            w_up=torch.cat((sd[b + f"mlp{s}.gate_proj.weight"], sd[b + f"mlp{s}.up_proj.weight"]), 0),
            w_down=sd[b + f"mlp{s}.down_proj.weight"]))
    return out


# ----------------------------------------------------------------------------- fp32 oracle
class TorchHalo:
    """Plain PyTorch statement: weights chosen row by row in the chunk's own order."""

    def __init__(self, cfg: HaloConfig, sd: Dict[str, torch.Tensor], mode: str = "act", *, dtype=torch.float32, device="cpu"):
        self.cfg, self.mode, self.dtype, self.device = cfg, mode, dtype, torch.device(device)
        self.sd = {k: v.to(self.device, dtype) for k, v in sd.items()}

    def _rms(self, t, w):
        tf = t.float()
        return (tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * w.float()).to(self.dtype)

    def _rope(self, t, pos: int):
        cfg = self.cfg
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32, device=self.device) / cfg.head_dim))
        ang = float(pos) * inv
        cos, sin = torch.cat((ang.cos(), ang.cos())), torch.cat((ang.sin(), ang.sin()))
        h = t.shape[-1] // 2
        return (t.float() * cos + torch.cat((-t[..., h:], t[..., :h]), -1).float() * sin).to(t.dtype)

    def input_rows(self, x: torch.Tensor, t: float, position_ids: torch.Tensor, text_ids: torch.Tensor) -> torch.Tensor:
        cfg, sd = self.cfg, self.sd
        n = x.shape[0]
        temb = _time_mlp(sd, cfg, self.mode, torch.full((n,), t))
        if self.mode == "act":
            body = F.linear(x.float(), sd["input_linear_layer.weight"].float(), sd["input_linear_layer.bias"].float()) + temb \
                + sinusoidal_pos_embedding(position_ids, cfg).to(self.device)
        else:
            body = F.linear(x.float(), sd["vae2llm.weight"].float(), sd["vae2llm.bias"].float()) + temb \
                + sd["latent_pos_embed.pos_embed"].float()[position_ids.long()]
        emb = sd[MODEL_P + "embed_tokens.weight"].float()[text_ids.long()]
        return torch.cat((emb[0:1], body, emb[1:2]), 0).to(self.dtype)

    @torch.no_grad()
    def decoder(self, rows: torch.Tensor, prefix_kv, rope_position: int) -> torch.Tensor:
        """``rows [n, H]`` in chunk order (text, twin rows, text) -> final-normed hidden ``[n, H]``."""
        cfg, sd, s = self.cfg, self.sd, SUFFIX[self.mode]
        n, hd, G = rows.shape[0], cfg.head_dim, cfg.heads // cfg.kv_heads
        is_twin = torch.ones(n, dtype=torch.bool, device=self.device)
        is_twin[0] = is_twin[-1] = False
        pick = lambda f: torch.where(is_twin.view(-1, *([1] * (f("").dim() - 1))), f(s), f(""))
        h = rows
        for i in range(cfg.layers):
            b = f"{LAYERS_P}{i}."
            y = pick(lambda z: self._rms(h, sd[b + f"input_layernorm{z}.weight"]))
            proj = lambda nm, heads: pick(lambda z: F.linear(y, sd[b + f"self_attn.{nm}_proj{z}.weight"],
                                                             sd[b + f"self_attn.{nm}_proj{z}.bias"])).view(n, heads, hd)
            q, k, v = proj("q", cfg.heads), proj("k", cfg.kv_heads), proj("v", cfg.kv_heads)
            q = pick(lambda z: self._rms(q, sd[b + f"self_attn.q_norm{z}.weight"]))
            k = pick(lambda z: self._rms(k, sd[b + f"self_attn.k_norm{z}.weight"]))
            q, k = self._rope(q, rope_position), self._rope(k, rope_position)
            pk, pv = prefix_kv[i]
            ka = torch.cat((pk.to(self.device, self.dtype).transpose(0, 1), k), 0).repeat_interleave(G, 1)
            va = torch.cat((pv.to(self.device, self.dtype).transpose(0, 1), v), 0).repeat_interleave(G, 1)
            sc = torch.einsum("qhd,khd->hqk", q.float(), ka.float()) / math.sqrt(hd)
            o = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), va.float()).to(self.dtype).reshape(n, -1)
            h = h + pick(lambda z: F.linear(o, sd[b + f"self_attn.o_proj{z}.weight"]))
            y = pick(lambda z: self._rms(h, sd[b + f"post_attention_layernorm{z}.weight"]))
            h = h + pick(lambda z: F.linear(F.silu(F.linear(y, sd[b + f"mlp{z}.gate_proj.weight"])) * F.linear(y, sd[b + f"mlp{z}.up_proj.weight"]),
                                            sd[b + f"mlp{z}.down_proj.weight"]))
        return pick(lambda z: self._rms(h, sd[MODEL_P + f"norm{z}.weight"]))

    @torch.no_grad()
    def rollout(self, prefix_kv, rope_position: int, x0: torch.Tensor, position_ids: torch.Tensor, text_ids: torch.Tensor,
                num_timesteps: int = 10) -> torch.Tensor:
        sd = self.sd
        ow, ob = ("output_linear_layer.weight", "output_linear_layer.bias") if self.mode == "act" else ("llm2vae.weight", "llm2vae.bias")
        x = x0.float().to(self.device)
        ts, dts = euler_schedule(num_timesteps)
        for t, dt in zip(ts.tolist(), dts.tolist()):
            hidden = self.decoder(self.input_rows(x, t, position_ids, text_ids), prefix_kv, rope_position)
            v = F.linear(hidden[1:-1].float(), sd[ow].float(), sd[ob].float())
            x = x - v * dt
        return x


    @torch.no_grad()
    def rollout_cfg(self, branches: Sequence[Optional[Tuple[Sequence, int]]], x0: torch.Tensor, position_ids: torch.Tensor,
                    text_ids: torch.Tensor, num_timesteps: int = 10, *, cfg_text_scale: float = 1.0, cfg_img_scale: float = 1.0,
                    cfg_renorm_min: float = 0.0, cfg_renorm_type: str = "global") -> torch.Tensor:
        """``branches = [cond, cfg_text, cfg_img]``, each ``(prefix_kv, rope_position)`` or ``None``: classifier-free guidance
        over the three prefix banks, then the norm of the guided velocity is capped at the conditional one."""
        sd = self.sd
        ow, ob = ("output_linear_layer.weight", "output_linear_layer.bias") if self.mode == "act" else ("llm2vae.weight", "llm2vae.bias")
        x = x0.float().to(self.device)
        ts, dts = euler_schedule(num_timesteps)
        for t, dt in zip(ts.tolist(), dts.tolist()):
            rows = self.input_rows(x, t, position_ids, text_ids)
            vel = lambda b: F.linear(self.decoder(rows, b[0], b[1])[1:-1].float(), sd[ow].float(), sd[ob].float())
            v = vel(branches[0])
            x = x - cfg_combine(v, vel(branches[1]) if cfg_text_scale > 1.0 else None, vel(branches[2]) if cfg_img_scale > 1.0 else None,
                                cfg_text_scale, cfg_img_scale, cfg_renorm_min, cfg_renorm_type) * dt
        return x


def cfg_combine(v: torch.Tensor, v_text: Optional[torch.Tensor], v_img: Optional[torch.Tensor], text_scale: float, img_scale: float,
                renorm_min: float = 0.0, renorm_type: str = "global") -> torch.Tensor:
    """Text guidance, then image guidance, then the result is scaled back so that its norm (whole tensor or per row) does
    not exceed the conditional velocity's (scale clamped to ``[renorm_min, 1]``).  With both scales at most 1 the
    conditional velocity passes through."""
    if text_scale <= 1.0 and img_scale <= 1.0:
        return v
    g = v
    if text_scale > 1.0:
        if v_text is None:
            raise ValueError("cfg_text_scale > 1 needs the cfg_text branch")
        g = v_text + text_scale * (v - v_text)
    if img_scale > 1.0:
        if v_img is None:
            raise ValueError("cfg_img_scale > 1 needs the cfg_img branch")
        g = v_img + img_scale * (g - v_img)
    if renorm_type == "global":
        n0, n1 = torch.linalg.vector_norm(v.float()), torch.linalg.vector_norm(g.float())
    elif renorm_type == "channel":
        n0, n1 = torch.linalg.vector_norm(v.float(), dim=-1, keepdim=True), torch.linalg.vector_norm(g.float(), dim=-1, keepdim=True)
    else:
        raise NotImplementedError(f"cfg_renorm_type {renorm_type!r} (global or channel)")
    return (g.float() * (n0 / (n1 + 1e-8)).clamp(min=renorm_min, max=1.0)).to(g.dtype)


# ----------------------------------------------------------------------------- device engine
class HaloEngine:
    """The twin-weight decoder over a paged prefix cache for one mode (``"act"``: action expert, ``"gen"``: image-flow
    step).  ``rollout`` returns the denoised ``[rows, action_dim | latent_dim]`` in a buffer the next call overwrites."""

    def __init__(self, cfg: HaloConfig, sd: Dict[str, torch.Tensor], mode: str = "act", *, max_prefix: int = 1024, device="cuda",
                 dtype=torch.float16, branches: int = 1):
        """``branches``: how many prefix banks the cache holds (3 for classifier-free guidance: cond, cfg_text, cfg_img)."""
        from ..ops import kernels as K
        from ..runtime.kv_cache import PagedKV
        from ..runtime.stack import NativeStack, StackSpec
        if mode not in SUFFIX:
            raise ValueError(f"mode must be 'act' or 'gen', got {mode!r}")
        self.K, self.cfg, self.mode, self.device, self.dtype = K, cfg, mode, torch.device(device), dtype
        dev, n, H = self.device, cfg.chunk_rows(mode), cfg.hidden
        self.n, self.body = n, n - 2
        self.max_prefix = max_prefix
        self.max_seq = (max_prefix + n + 15) // 16 * 16
        self.branches = branches
        self.cache = PagedKV(cfg.layers, branches, self.max_seq, cfg.kv_heads, cfg.head_dim, device=device, dtype=dtype)
        self.cache.reserve_all()
        s = SUFFIX[mode]
        self.stack = NativeStack(
            StackSpec(layers=cfg.layers, hidden=H, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, inter=cfg.inter,
                      norm="rms", mlp="swiglu", eps=cfg.eps, qk_norm=True, rot_dim=cfg.head_dim, paged_kv=True, causal=False,
                      max_tokens=(n + 15) // 16 * 16, max_seqs=1),
            _branch_layers(sd, cfg, ""), device=device, dtype=dtype, kv_cache=self.cache,
            final_norm_w=sd[MODEL_P + "norm.weight"], twin_layer_weights=_branch_layers(sd, cfg, s),
            twin_final_norm_w=sd[MODEL_P + f"norm{s}.weight"])
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32) / cfg.head_dim))
        self._inv = inv
        self.width = cfg.action_dim if mode == "act" else cfg.latent_dim
        self.w_pad = (self.width + 7) // 8 * 8
        keep = [k for k, _, _ in halo_shapes(cfg, mode) if not k.startswith(LAYERS_P) and not k.startswith(MODEL_P + "norm")]
        self._small = {k: sd[k].to(dev, torch.float32) for k in keep}
        self._schedules: Dict[int, dict] = {}
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        i32 = dict(dtype=torch.int32, device=dev)
        self.x = torch.zeros(self.body, self.w_pad, dtype=dtype, device=dev)
        self.h = torch.zeros(n, H, dtype=dtype, device=dev)            # rows ordered [text, text, body...]
        self.hn = torch.zeros(n, H, dtype=dtype, device=dev)
        self.row_bias = torch.zeros(self.body, H, dtype=dtype, device=dev)     # position term of the body rows
        self.text_rows = torch.zeros(2, H, dtype=dtype, device=dev)
        self.s_pos = torch.zeros(n, **i32)
        # stack row r -> chunk row: text rows 0 and n-1 first, then the body rows 1 .. n-2
        self.chunk_row = torch.cat((torch.tensor([0, n - 1]), torch.arange(1, n - 1))).to(torch.int32)
        self.s_cache_pos = torch.zeros(n, **i32)
        self.s_seq = torch.zeros(n, **i32)
        self.s_qstart = torch.zeros(1, **i32)
        self.s_qlen = torch.full((1,), n, **i32)
        self.s_kvlen = torch.zeros(1, **i32)
        self.cos = torch.zeros(branches, cfg.head_dim // 2, dtype=torch.float32, device=dev)
        self.sin = torch.zeros(branches, cfg.head_dim // 2, dtype=torch.float32, device=dev)
        self.prefix_len = 0
        # per-bank row metadata of the guidance branches (bank 0 is the plain path's)
        self.b_pos = [torch.full((n,), b, **i32) for b in range(branches)]
        self.b_cache_pos = [torch.zeros(n, **i32) for _ in range(branches)]
        self.b_kvlen = [torch.zeros(1, **i32) for _ in range(branches)]
        self.b_ready = [False] * branches
        if branches > 1:
            self.h0 = torch.zeros(n, H, dtype=dtype, device=dev)
            self.vel = [torch.zeros(self.body, self.w_pad, dtype=dtype, device=dev) for _ in range(branches)]

    # ------------------------------------------------------------------ prefix
    @torch.no_grad()
    def set_prefix(self, prefix_kv: Sequence[Tuple[torch.Tensor, torch.Tensor]], rope_position: int, *, branch: int = 0) -> int:
        """Copy the prefix's rotated keys / values (``[kv_heads, P, head_dim]`` per layer) into bank ``branch`` of the cache;
        every row of the chunk then rotates at ``rope_position`` when it runs against that bank."""
        cfg, dev = self.cfg, self.device
        if not 0 <= branch < self.branches:
            raise ValueError(f"branch {branch} is outside the engine's {self.branches} banks")
        P = int(prefix_kv[0][0].shape[1])
        if P > self.max_prefix or len(prefix_kv) != cfg.layers:
            raise ValueError(f"prefix of {P} rows / {len(prefix_kv)} layers does not fit (max_prefix {self.max_prefix}, {cfg.layers} layers)")
        for i, (k, v) in enumerate(prefix_kv):
            self.cache.scatter(i, branch, k, v, 0)
        self.cache.sync_table()
        ang = float(rope_position) * self._inv
        self.cos[branch].copy_(ang.cos().to(dev))
        self.sin[branch].copy_(ang.sin().to(dev))
        self.b_cache_pos[branch].copy_((self.chunk_row + P).to(dev))
        self.b_kvlen[branch].fill_(P + self.n)
        self.b_ready[branch] = True
        if branch == 0:
            self.s_cache_pos.copy_(self.b_cache_pos[0])
            self.s_kvlen.copy_(self.b_kvlen[0])
            self.prefix_len = P
        return P

    # ------------------------------------------------------------------ schedule
    def schedule(self, num_timesteps: int) -> dict:
        hit = self._schedules.get(num_timesteps)
        if hit is not None:
            return hit
        cfg, sd = self.cfg, self._small
        ts, dts = euler_schedule(num_timesteps)
        iw, ib, ow, ob = (("input_linear_layer.weight", "input_linear_layer.bias", "output_linear_layer.weight", "output_linear_layer.bias")
                          if self.mode == "act" else ("vae2llm.weight", "vae2llm.bias", "llm2vae.weight", "llm2vae.bias"))
        temb = _time_mlp(sd, cfg, self.mode, ts)                                       # [steps, H]
        pad = lambda m, rows, cols: F.pad(m, (0, cols - m.shape[1], 0, rows - m.shape[0]))
        # one output projection per step: -dt_k folded in, so that x + GEMM is the Euler update
        out_w = torch.stack([pad(sd[ow] * -float(d), self.w_pad, cfg.hidden) for d in dts]).to(self.dtype).contiguous()
        out_b = torch.stack([F.pad(sd[ob] * -float(d), (0, self.w_pad - self.width)) for d in dts]).to(self.dtype).contiguous()
        hit = dict(steps=int(ts.numel()), in_w=pad(sd[iw], cfg.hidden, self.w_pad).to(self.dtype).contiguous(),
                   step_bias=(temb + sd[ib][None]).to(self.dtype).contiguous(), out_w=out_w, out_b=out_b,
                   out_w_plain=pad(sd[ow], self.w_pad, cfg.hidden).to(self.dtype).contiguous(),
                   out_b_plain=F.pad(sd[ob], (0, self.w_pad - self.width)).to(self.dtype).contiguous())
        self._schedules[num_timesteps] = hit
        return hit

    def _loop(self, num_timesteps: int) -> None:
        K, sch = self.K, self.schedule(num_timesteps)
        n = self.n
        for k in range(sch["steps"]):
            # body rows: in_proj(x) + (time term of step k) + (position term of the row); text rows are constants
            K.gemm(self.x, sch["in_w"], bias=sch["step_bias"][k], residual=self.row_bias, out=self.h[2:])
            self.h[:2].copy_(self.text_rows)
            self.stack.forward(self.h, q_start=self.s_qstart, q_len=self.s_qlen, kv_len=self.s_kvlen, max_q_len=n,
                               max_kv_len=self.max_seq, pos=self.s_pos, cos=self.cos, sin=self.sin, seq_of_tok=self.s_seq,
                               cache_pos=self.s_cache_pos, page_table=self.cache.page_table, twin_split=2)
            self.stack.final_norm_twin(self.h, 2, out=self.hn)
            K.gemm(self.hn[2:], sch["out_w"][k], bias=sch["out_b"][k], residual=self.x, out=self.x)     # x <- x - dt * v

    def _loop_cfg(self, num_timesteps: int, text_scale: float, img_scale: float, renorm_min: float, renorm_type: str) -> None:
        """The guided loop: every step runs the chunk against the banks its scales ask for (the input rows are built once),
        combines the velocities and applies the Euler update."""
        K, sch = self.K, self.schedule(num_timesteps)
        n = self.n
        use = [0] + ([1] if text_scale > 1.0 else []) + ([2] if img_scale > 1.0 else [])
        ts, dts = euler_schedule(num_timesteps)
        ow, ob = sch["out_w_plain"], sch["out_b_plain"]
        for k in range(sch["steps"]):
            K.gemm(self.x, sch["in_w"], bias=sch["step_bias"][k], residual=self.row_bias, out=self.h0[2:])
            self.h0[:2].copy_(self.text_rows)
            for b in use:
                self.h.copy_(self.h0)
                self.stack.forward(self.h, q_start=self.s_qstart, q_len=self.s_qlen, kv_len=self.b_kvlen[b], max_q_len=n,
                                   max_kv_len=self.max_seq, pos=self.b_pos[b], cos=self.cos, sin=self.sin, seq_of_tok=self.s_seq,
                                   cache_pos=self.b_cache_pos[b], page_table=self.cache.page_table[b:b + 1], twin_split=2)
                self.stack.final_norm_twin(self.h, 2, out=self.hn)
                K.gemm(self.hn[2:], ow, bias=ob, out=self.vel[b])
            v = cfg_combine(self.vel[0], self.vel[1] if 1 in use else None, self.vel[2] if 2 in use else None, text_scale, img_scale,
                            renorm_min, renorm_type)
            self.x.add_(v, alpha=-float(dts[k]))

    @torch.no_grad()
    def rollout(self, x0: torch.Tensor, position_ids: torch.Tensor, text_ids: torch.Tensor, num_timesteps: int = 10, *,
                use_graph: bool = True, cfg_text_scale: float = 1.0, cfg_img_scale: float = 1.0, cfg_renorm_min: float = 0.0,
                cfg_renorm_type: str = "global") -> torch.Tensor:
        """With a guidance scale above 1 the chunk also runs against bank 1 (``cfg_text``) / bank 2 (``cfg_img``), set with
        ``set_prefix(..., branch=)``, and the velocities are combined by :func:`cfg_combine`."""
        cfg, dev = self.cfg, self.device
        guided = cfg_text_scale > 1.0 or cfg_img_scale > 1.0
        if guided:
            need = [0] + ([1] if cfg_text_scale > 1.0 else []) + ([2] if cfg_img_scale > 1.0 else [])
            if max(need) >= self.branches or not all(self.b_ready[b] for b in need):
                raise ValueError(f"guidance needs prefix banks {need}: build the engine with branches=3 and call set_prefix(..., branch=) for each")
            if cfg_renorm_type not in ("global", "channel"):
                raise NotImplementedError(f"cfg_renorm_type {cfg_renorm_type!r} (global or channel)")
        if tuple(x0.shape) != (self.body, self.width):
            raise ValueError(f"x0 must be {(self.body, self.width)}, got {tuple(x0.shape)}")
        if self.mode == "act":
            pos_term = sinusoidal_pos_embedding(position_ids.flatten().cpu(), cfg)
        else:
            pos_term = self._small["latent_pos_embed.pos_embed"][position_ids.flatten().long().to(dev)]
        self.row_bias.copy_(pos_term.to(dev, self.dtype))
        self.text_rows.copy_(self._small[MODEL_P + "embed_tokens.weight"][text_ids.flatten().long().to(dev)].to(self.dtype))
        self.x.zero_()
        self.x[:, :self.width].copy_(x0.to(dev, self.dtype))
        run = (lambda steps: self._loop_cfg(steps, cfg_text_scale, cfg_img_scale, cfg_renorm_min, cfg_renorm_type)) if guided \
            else self._loop
        key = (num_timesteps, cfg_text_scale, cfg_img_scale, cfg_renorm_min, cfg_renorm_type) if guided else num_timesteps
        if not use_graph:
            run(num_timesteps)
        else:
            gph = self._graphs.get(key)
            if gph is None:
                snap = self.x.clone()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    run(2)                                             # warm-up: one step
                torch.cuda.current_stream().wait_stream(s)
                self.schedule(num_timesteps)
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph, stream=s):
                    run(num_timesteps)
                torch.cuda.synchronize()
                self.x.copy_(snap)
                self._graphs[key] = gph
            gph.replay()
        return self.x[:, :self.width]

    def check_status(self) -> None:
        self.stack.check_status()

    def close(self) -> None:
        self._graphs.clear()
        self.stack.close()
        self.cache.close()


__all__ = ["HaloConfig", "HaloEngine", "TorchHalo", "cfg_combine", "tiny_halo_config", "halo_shapes", "random_halo_state_dict",
           "timestep_embedding", "sinusoidal_pos_embedding", "euler_schedule", "SUFFIX"]
