"""LingBot-VLA-v2: a Qwen3-VL prefix and a sparse-MoE flow-matching action expert that share one KV cache.

Data flow of one action chunk:

  camera images + instruction tokens -> Qwen3-VL (vision tower, DeepStack, M-RoPE text decoder), one packed
  prefill: K/V of every decoder layer land in the paged cache at rows [0, S)
  noise x_1 [horizon, action_dim]; for k in 0..num_steps-1 (t_0 = 1, t_{k+1} = t_k + dt, dt = -1/num_steps):
      suffix rows: [ state_proj(state) | mlp_out(silu(W_a(action_in(x)) + W_t sincos(t_k) + b)) ]     (1 + horizon rows)
      expert layer i (36 layers, width 768, the prefix decoder's head geometry):
          FiLM RMSNorm  y = norm(h) * ((1 + gamma_i(c_k)) * w_i) + beta_i(c_k),  c_k = sincos(t_k)
          q/k/v (+bias) -> RoPE at p0 + row (p0 = largest prefix position + 1) -> K/V written at cache rows S + row
          attention over [prefix rows | suffix rows] under the suffix mask -> o_proj -> h += o
          FiLM RMSNorm -> sparse MoE MLP (sigmoid router + selection-only bias, top-4 of 32, normalised, x4,
          plus the always-on shared expert) -> h += mlp
      v = action_out_proj(rmsnorm(h)[1:]);  x <- x + dt * v

Suffix mask: the state row sees the prefix and itself; every action row sees the prefix, the state row and all
action rows; the last ``blocked_tail`` prefix rows (learned future-depth query tokens, when a checkpoint has them)
are hidden from the whole suffix.

Everything that depends on the time step only is computed once per ``num_steps``: the FiLM scale/shift of every
(step, layer, norm), the time half of the suffix encoder (folded into a per-step bias) and the product of the two
consecutive input projections.  ``dt`` is folded into the output projection, so the Euler update is that GEMM's
residual epilogue, and the whole loop replays from one CUDA graph whose per-call values (prefix length, positions,
mask, page table) live in device buffers at fixed addresses.

Reference behaviour: ``python/rpu_backend/adapters/lingbot_vla_v2/runtime.py:582-700,2598-2740`` (suffix encoder,
FiLM fold, mask, Euler loop), ``adapters/lingbot_vla_v2/convert.py:36-160`` (geometry and checkpoint names),
``src/fused/rpu_lingbot_v2_moe_model.h:24-49`` (router math), ``.cpp:1029-1511`` (MoE MLP).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

VLM_P = "model.qwenvl_with_expert.qwenvl."
EXP_P = "model.qwenvl_with_expert.qwen_expert.model."
HEAD_NAMES = ("model.state_proj", "model.action_in_proj", "model.action_out_proj", "model.action_time_mlp_in",
              "model.action_time_mlp_out")


@dataclass
class Lingbot2Config:
    hidden: int = 768
    layers: int = 36
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    eps: float = 1e-6
    rope_theta: float = 5e6
    experts: int = 32
    top_k: int = 4
    routed_inter: int = 512
    shared_inter: int = 704
    routed_scale: float = 4.0
    horizon: int = 50
    action_dim: int = 55
    state_dim: int = 55
    num_steps: int = 10
    min_period: float = 4e-3
    max_period: float = 4.0
    blocked_tail: int = 0        # trailing prefix rows hidden from the suffix

    @property
    def suffix_rows(self) -> int:
        return 1 + self.horizon


def tiny_lingbot2_config(**kw) -> Lingbot2Config:
    base = dict(hidden=64, layers=4, heads=2, kv_heads=1, head_dim=64, rope_theta=1e4, experts=8, top_k=2,
                routed_inter=32, shared_inter=40, routed_scale=2.0, horizon=6, action_dim=7, state_dim=5, num_steps=4)
    base.update(kw)
    return Lingbot2Config(**base)


def lingbot2_expert_shapes(cfg: Lingbot2Config) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """(checkpoint name, shape, kind) of every tensor of the action expert and the action head."""
    H, E, I, S = cfg.hidden, cfg.experts, cfg.routed_inter, cfg.shared_inter
    for i in range(cfg.layers):
        b = f"{EXP_P}layers.{i}."
        for n, rows in (("q", cfg.heads), ("k", cfg.kv_heads), ("v", cfg.kv_heads)):
            yield b + f"self_attn.{n}_proj.weight", (rows * cfg.head_dim, H), "matrix"
            yield b + f"self_attn.{n}_proj.bias", (rows * cfg.head_dim,), "bias"
        yield b + "self_attn.o_proj.weight", (H, cfg.heads * cfg.head_dim), "matrix"
        for n in ("input_layernorm", "post_attention_layernorm"):
            yield b + n + ".weight", (H,), "norm"
            for m in ("gamma", "beta"):
                yield b + f"{n}.{m}.weight", (H, H), "matrix"
                yield b + f"{n}.{m}.bias", (H,), "bias"
        yield b + "mlp.gate.weight", (E, H), "router"
        yield b + "mlp.e_score_correction_bias", (E,), "bias"
        yield b + "mlp.experts.gate_proj", (E, I, H), "matrix"
        yield b + "mlp.experts.up_proj", (E, I, H), "matrix"
        yield b + "mlp.experts.down_proj", (E, H, I), "matrix"
        yield b + "mlp.shared_expert.gate_proj.weight", (S, H), "matrix"
        yield b + "mlp.shared_expert.up_proj.weight", (S, H), "matrix"
        yield b + "mlp.shared_expert.down_proj.weight", (H, S), "matrix"
    yield EXP_P + "norm.weight", (H,), "norm"
    yield "model.state_proj.weight", (H, cfg.state_dim), "matrix"
    yield "model.state_proj.bias", (H,), "bias"
    yield "model.action_in_proj.weight", (H, cfg.action_dim), "matrix"
    yield "model.action_in_proj.bias", (H,), "bias"
    yield "model.action_out_proj.weight", (cfg.action_dim, H), "matrix"
    yield "model.action_out_proj.bias", (cfg.action_dim,), "bias"
    yield "model.action_time_mlp_in.weight", (H, 2 * H), "matrix"
    yield "model.action_time_mlp_in.bias", (H,), "bias"
    yield "model.action_time_mlp_out.weight", (H, H), "matrix"
    yield "model.action_time_mlp_out.bias", (H,), "bias"


def random_lingbot2_expert(cfg: Lingbot2Config, *, seed: int = 0, std: float = 0.05, dtype=torch.float16,
                           device="cpu") -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in lingbot2_expert_shapes(cfg):
        r = torch.randn(shape, generator=g)
        t = {"matrix": r * std, "router": r * 0.3, "norm": 1.0 + 0.05 * r, "bias": 0.03 * r}[kind]
        sd[name] = t.to(device, dtype)
    return sd


def sinusoidal_embedding(t: torch.Tensor, dim: int, min_period: float, max_period: float) -> torch.Tensor:
    """``[n] -> [n, dim]`` fp32: sin | cos over ``dim / 2`` log-spaced periods."""
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float32)
    period = min_period * (max_period / min_period) ** frac
    ang = (2.0 * math.pi / period)[None, :] * t.float()[:, None]
    return torch.cat((ang.sin(), ang.cos()), 1)


def euler_times(num_steps: int) -> List[float]:
    """``t_0 = 1`` and ``t_{k+1} = t_k + dt`` accumulated step by step (the order the policy was trained with)."""
    out, t = [], 1.0
    for _ in range(num_steps):
        out.append(t)
        t += -1.0 / num_steps
    return out


def suffix_mask(cfg: Lingbot2Config, prefix_len: int, width: int) -> torch.Tensor:
    """Boolean ``[suffix_rows, width]``: which cache rows each suffix row attends to (cache row = prefix row, then the
    state row at ``prefix_len``, then the action rows)."""
    n = cfg.suffix_rows
    m = torch.zeros(n, width, dtype=torch.bool)
    m[:, :max(0, prefix_len - cfg.blocked_tail)] = True
    m[0, prefix_len] = True
    m[1:, prefix_len:prefix_len + n] = True
    return m


def film_schedule(sd: Dict[str, torch.Tensor], cfg: Lingbot2Config, num_steps: int) -> torch.Tensor:
    """``[num_steps, layers, 2, 3 * hidden]`` fp32 rows ``[scale | shift | 0]`` for the stack's modulated RMSNorm
    ``norm(h) * (1 + scale) + shift``: ``scale = (1 + gamma(c)) * w - 1``, ``shift = beta(c)``, ``c = sincos(t_k)``."""
    H = cfg.hidden
    cond = sinusoidal_embedding(torch.tensor(euler_times(num_steps)), H, cfg.min_period, cfg.max_period)
    dev = sd[EXP_P + "norm.weight"].device
    cond = cond.to(dev)
    out = torch.zeros(num_steps, cfg.layers, 2, 3 * H, dtype=torch.float32, device=dev)
    for i in range(cfg.layers):
        for j, n in enumerate(("input_layernorm", "post_attention_layernorm")):
            p = f"{EXP_P}layers.{i}.{n}"
            w = sd[p + ".weight"].float()
            gamma = F.linear(cond, sd[p + ".gamma.weight"].float(), sd[p + ".gamma.bias"].float())
            beta = F.linear(cond, sd[p + ".beta.weight"].float(), sd[p + ".beta.bias"].float())
            out[:, i, j, :H] = (1.0 + gamma) * w - 1.0
            out[:, i, j, H:2 * H] = beta
    return out


def folded_suffix_encoder(sd: Dict[str, torch.Tensor], cfg: Lingbot2Config, num_steps: int):
    """``(W_fused [hidden, action_dim], step_bias [num_steps, hidden])`` fp32 with
    ``silu(x @ W_fused.T + step_bias[k]) == silu(mlp_in(cat(action_in(x), sincos(t_k))))``: the two linears before the
    nonlinearity collapse into one, and everything that only depends on ``t_k`` into a bias."""
    H = cfg.hidden
    win, b_in = sd["model.action_time_mlp_in.weight"].float(), sd["model.action_time_mlp_in.bias"].float()
    wa, wt = win[:, :H], win[:, H:]
    wp, bp = sd["model.action_in_proj.weight"].float(), sd["model.action_in_proj.bias"].float()
    temb = sinusoidal_embedding(torch.tensor(euler_times(num_steps)), H, cfg.min_period, cfg.max_period).to(win.device)
    return (wa @ wp).contiguous(), (F.linear(temb, wt, b_in) + F.linear(bp, wa)[None]).contiguous()


# ----------------------------------------------------------------------------- fp32 oracle of the expert
class TorchLingbot2Expert:
    """Plain PyTorch statement of the denoise loop over given prefix K/V (``[layers] x (K, V)`` of shape
    ``[kv_heads, S, head_dim]``, already rotated), written without any of the engine's folds."""

    def __init__(self, cfg: Lingbot2Config, sd: Dict[str, torch.Tensor], *, dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.sd = {k: v.to(self.device, dtype) for k, v in sd.items()}

    def _rope(self, t, pos):      # t [heads, n, hd]
        cfg = self.cfg
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32, device=self.device) / cfg.head_dim))
        ang = pos.float()[None, :, None] * inv
        cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)
        h = t.shape[-1] // 2
        return (t.float() * cos + torch.cat((-t[..., h:], t[..., :h]), -1).float() * sin).to(t.dtype)

    def _moe(self, b: str, x: torch.Tensor) -> torch.Tensor:
        cfg, sd = self.cfg, self.sd
        logits = x.float() @ sd[b + "mlp.gate.weight"].float().t()
        sc = torch.sigmoid(logits)
        top = torch.topk(sc + sd[b + "mlp.e_score_correction_bias"].float(), cfg.top_k, -1).indices
        w = torch.gather(sc, 1, top)
        w = w / (w.sum(-1, keepdim=True) + 1e-20) * cfg.routed_scale
        xf = x.float()
        out = (F.silu(xf @ sd[b + "mlp.shared_expert.gate_proj.weight"].float().t()) *
               (xf @ sd[b + "mlp.shared_expert.up_proj.weight"].float().t())) @ sd[b + "mlp.shared_expert.down_proj.weight"].float().t()
        for e in range(cfg.experts):
            rows, pick = (top == e).nonzero(as_tuple=True)
            if rows.numel():
                h = F.silu(xf[rows] @ sd[b + "mlp.experts.gate_proj"][e].float().t()) * (xf[rows] @ sd[b + "mlp.experts.up_proj"][e].float().t())
                out[rows] += w[rows, pick][:, None] * (h @ sd[b + "mlp.experts.down_proj"][e].float().t())
        return out.to(x.dtype)

    @torch.no_grad()
    def sample_actions(self, prefix_kv, prefix_len: int, p0: int, state: torch.Tensor, noise: torch.Tensor,
                       num_steps: Optional[int] = None) -> torch.Tensor:
        cfg, sd = self.cfg, self.sd
        num_steps = num_steps or cfg.num_steps
        n, H, hd = cfg.suffix_rows, cfg.hidden, cfg.head_dim
        G = cfg.heads // cfg.kv_heads
        x = noise.to(self.device, self.dtype)
        dt = -1.0 / num_steps
        state_emb = F.linear(state.to(self.device, self.dtype), sd["model.state_proj.weight"], sd["model.state_proj.bias"])
        mask = suffix_mask(cfg, prefix_len, prefix_len + n).to(self.device)
        pos = p0 + torch.arange(n, device=self.device)

        def rms(t):
            tf = t.float()
            return tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + cfg.eps)
        for t in euler_times(num_steps):
            temb = sinusoidal_embedding(torch.tensor([t]), H, cfg.min_period, cfg.max_period).to(self.device, self.dtype)
            a = F.linear(x, sd["model.action_in_proj.weight"], sd["model.action_in_proj.bias"])
            a = F.silu(F.linear(torch.cat((a, temb.expand(a.shape[0], -1)), -1), sd["model.action_time_mlp_in.weight"],
                                sd["model.action_time_mlp_in.bias"]))
            a = F.linear(a, sd["model.action_time_mlp_out.weight"], sd["model.action_time_mlp_out.bias"])
            h = torch.cat((state_emb[None], a), 0)
            for i in range(cfg.layers):
                b = f"{EXP_P}layers.{i}."

                def film(name, v):
                    p = b + name
                    gamma = F.linear(temb, sd[p + ".gamma.weight"], sd[p + ".gamma.bias"]).float()
                    beta = F.linear(temb, sd[p + ".beta.weight"], sd[p + ".beta.bias"]).float()
                    return (rms(v) * ((1.0 + gamma) * sd[p + ".weight"].float()) + beta).to(self.dtype)
                y = film("input_layernorm", h)
                q = F.linear(y, sd[b + "self_attn.q_proj.weight"], sd[b + "self_attn.q_proj.bias"]).view(n, cfg.heads, hd).transpose(0, 1)
                k = F.linear(y, sd[b + "self_attn.k_proj.weight"], sd[b + "self_attn.k_proj.bias"]).view(n, cfg.kv_heads, hd).transpose(0, 1)
                v = F.linear(y, sd[b + "self_attn.v_proj.weight"], sd[b + "self_attn.v_proj.bias"]).view(n, cfg.kv_heads, hd).transpose(0, 1)
                q, k = self._rope(q, pos), self._rope(k, pos)
                kk = torch.cat((prefix_kv[i][0].to(self.device, self.dtype), k), 1).repeat_interleave(G, 0)
                vv = torch.cat((prefix_kv[i][1].to(self.device, self.dtype), v), 1).repeat_interleave(G, 0)
                s = (q.float() @ kk.float().transpose(-1, -2)) / math.sqrt(hd)
                s = s.masked_fill(~mask[None], float("-inf"))
                o = (torch.softmax(s, -1) @ vv.float()).to(self.dtype).transpose(0, 1).reshape(n, -1)
                h = h + F.linear(o, sd[b + "self_attn.o_proj.weight"])
                h = h + self._moe(b, film("post_attention_layernorm", h))
            hn = (rms(h) * sd[EXP_P + "norm.weight"].float()).to(self.dtype)
            v_t = F.linear(hn[1:], sd["model.action_out_proj.weight"], sd["model.action_out_proj.bias"])
            x = x + dt * v_t
        return x


# ----------------------------------------------------------------------------- device engine
class Lingbot2Engine:
    """Qwen3-VL prefix + MoE action expert on the accelerator.  ``predict(...)`` returns ``[horizon, action_dim]``
    in a stable buffer that the next call overwrites."""

    def __init__(self, cfg: Lingbot2Config, hf_vlm_config, get_weight: Callable[[str], torch.Tensor], *,
                 names: Optional[set] = None, device="cuda", dtype=torch.float16, max_prefix: int = 1024,
                 max_patches: int = 4096):
        from ..ops import kernels as K
        from ..runtime.stack import NativeStack, StackSpec
        from .qwen3_vl import Qwen3VLEngine
        self.K, self.cfg, self.device, self.dtype = K, cfg, torch.device(device), dtype
        dev = self.device
        n = cfg.suffix_rows
        self.max_prefix = max_prefix
        self.max_seq = (max_prefix + n + 15) // 16 * 16

        def vlm_get(name: str) -> torch.Tensor:
            return get_weight(VLM_P + name)
        vlm_names = None if names is None else {x[len(VLM_P):] for x in names if x.startswith(VLM_P)}
        self.vlm = Qwen3VLEngine(hf_vlm_config, vlm_get, names=vlm_names, device=device, dtype=dtype,
                                 max_seq_len=self.max_seq, max_batch=1, max_patches=max_patches,
                                 max_prefill_tokens=max(max_prefix, 256))
        t = self.vlm.cfg
        if (t.num_layers, t.num_kv_heads, t.head_dim) != (cfg.layers, cfg.kv_heads, cfg.head_dim):
            raise ValueError("prefix decoder and action expert must share the KV geometry (layers, kv heads, head_dim): "
                             f"{(t.num_layers, t.num_kv_heads, t.head_dim)} vs {(cfg.layers, cfg.kv_heads, cfg.head_dim)}")
        self.cache = self.vlm.text.cache
        g = get_weight
        E, I, S = cfg.experts, cfg.routed_inter, cfg.shared_inter
        layers = []
        for i in range(cfg.layers):
            b = f"{EXP_P}layers.{i}."
            gates, ups, downs = g(b + "mlp.experts.gate_proj"), g(b + "mlp.experts.up_proj"), g(b + "mlp.experts.down_proj")
            w_up = torch.cat((gates.reshape(E * I, -1), g(b + "mlp.shared_expert.gate_proj.weight"),
                              ups.reshape(E * I, -1), g(b + "mlp.shared_expert.up_proj.weight")), 0)
            w_down = torch.cat((downs.permute(1, 0, 2).reshape(cfg.hidden, E * I), g(b + "mlp.shared_expert.down_proj.weight")), 1)
            layers.append(dict(
                wqkv=torch.cat([g(b + f"self_attn.{x}_proj.weight") for x in "qkv"], 0),
                bqkv=torch.cat([g(b + f"self_attn.{x}_proj.bias") for x in "qkv"], 0),
                wo=g(b + "self_attn.o_proj.weight"), w_up=w_up, w_down=w_down,
                moe_router_w=g(b + "mlp.gate.weight"), moe_router_bias=g(b + "mlp.e_score_correction_bias")))
        self.inter = E * I + S
        self.expert = NativeStack(
            StackSpec(layers=cfg.layers, hidden=cfg.hidden, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
                      inter=self.inter, norm="adarms", mlp="swiglu", eps=cfg.eps, rot_dim=cfg.head_dim, paged_kv=True,
                      causal=False, max_tokens=(n + 15) // 16 * 16, max_seqs=1, moe_experts=E, moe_top_k=cfg.top_k,
                      moe_expert_inter=I, moe_score_fn="sigmoid", moe_norm_topk=True, moe_routed_scale=cfg.routed_scale),
            layers, device=device, dtype=dtype, kv_cache=self.cache)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32) / cfg.head_dim))
        ang = torch.arange(self.max_seq + 4096, dtype=torch.float32)[:, None] * inv[None]
        self.cos, self.sin = ang.cos().to(dev).contiguous(), ang.sin().to(dev).contiguous()
        keep = [x for x, _, _ in lingbot2_expert_shapes(cfg) if ".gamma." in x or ".beta." in x or "layernorm.weight" in x
                or x.startswith("model.") or x == EXP_P + "norm.weight"]
        self._small = {k: g(k).to(dev, torch.float32) for k in keep}
        self.final_norm_w = g(EXP_P + "norm.weight").to(dev, dtype).contiguous()
        self.state_w = g("model.state_proj.weight").to(dev, torch.float32)
        self.state_b = g("model.state_proj.bias").to(dev, torch.float32)
        self.ad_pad = (cfg.action_dim + 7) // 8 * 8           # GEMM K and N are multiples of 8
        self._schedules: Dict[int, dict] = {}
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        i32 = dict(dtype=torch.int32, device=dev)
        H = cfg.hidden
        self.x = torch.zeros(cfg.horizon, self.ad_pad, dtype=dtype, device=dev)
        self.h = torch.zeros(n, H, dtype=dtype, device=dev)
        self.hn = torch.zeros(n, H, dtype=dtype, device=dev)
        self.enc = torch.zeros(cfg.horizon, H, dtype=dtype, device=dev)
        self.state_emb = torch.zeros(1, H, dtype=dtype, device=dev)
        self.s_pos = torch.zeros(n, **i32)
        self.s_cache_pos = torch.zeros(n, **i32)
        self.s_seq = torch.zeros(n, **i32)
        self.s_qstart = torch.zeros(1, **i32)
        self.s_qlen = torch.full((1,), n, **i32)
        self.s_kvlen = torch.zeros(1, **i32)
        self.mask = torch.zeros(n, (self.max_seq + 127) // 128 * 128, dtype=torch.uint8, device=dev)[:, :self.max_seq]   # pitch: whole 128-key blocks
        self.image_token_id = self.vlm.image_token_id
        cg = lambda k, d: hf_vlm_config.get(k, d) if isinstance(hf_vlm_config, dict) else getattr(hf_vlm_config, k, d)
        self.vision_start_id, self.vision_end_id = int(cg("vision_start_token_id", 151652)), int(cg("vision_end_token_id", 151653))

    # ------------------------------------------------------------------ per-num_steps constants
    def schedule(self, num_steps: int) -> dict:
        hit = self._schedules.get(num_steps)
        if hit is not None:
            return hit
        cfg, sd = self.cfg, self._small
        film = film_schedule(sd, cfg, num_steps).view(num_steps, cfg.layers, 2, 1, 3 * cfg.hidden)
        wf, sb = folded_suffix_encoder(sd, cfg, num_steps)
        pad = lambda w, rows, cols: F.pad(w, (0, cols - w.shape[1], 0, rows - w.shape[0]))
        dt = -1.0 / num_steps
        hit = dict(
            film=film.to(self.dtype).contiguous(),
            enc_w=pad(wf, cfg.hidden, self.ad_pad).to(self.dtype).contiguous(),
            enc_b=sb.to(self.dtype).contiguous(),
            out_w_t=sd["model.action_time_mlp_out.weight"].to(self.dtype).contiguous(),
            out_b_t=sd["model.action_time_mlp_out.bias"].to(self.dtype).contiguous(),
            out_w=pad(sd["model.action_out_proj.weight"] * dt, self.ad_pad, cfg.hidden).to(self.dtype).contiguous(),
            out_b=F.pad(sd["model.action_out_proj.bias"] * dt, (0, self.ad_pad - cfg.action_dim)).to(self.dtype).contiguous())
        self._schedules[num_steps] = hit
        return hit

    # ------------------------------------------------------------------ prefix
    def build_input_ids(self, tokens_per_image: Sequence[int], lang_tokens: torch.Tensor, *,
                        vision_boundaries: bool = False, tail_token_id: Optional[int] = None) -> torch.Tensor:
        """Prefix id sequence: one run of image placeholders per camera (with ``vision_boundaries`` each run sits
        between a vision-start and a vision-end token), then the instruction tokens and, when ``tail_token_id`` is
        given, ``blocked_tail`` filler rows that stand in for learned query tokens the action rows must not see."""
        parts = []
        for t in tokens_per_image:
            run = torch.full((int(t),), self.image_token_id, dtype=torch.long)
            if vision_boundaries:
                run = torch.cat((torch.tensor([self.vision_start_id]), run, torch.tensor([self.vision_end_id])))
            parts.append(run)
        parts.append(lang_tokens.flatten().to(torch.long))
        if self.cfg.blocked_tail and tail_token_id is not None:
            parts.append(torch.full((self.cfg.blocked_tail,), int(tail_token_id), dtype=torch.long))
        return torch.cat(parts)

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor], image_grid_thw) -> Tuple[int, int]:
        """Fill the KV cache with the prefix; returns ``(prefix rows S, first suffix rope position p0)``."""
        S = int(input_ids.numel())
        if S > self.max_prefix:
            raise ValueError(f"prefix of {S} rows exceeds max_prefix {self.max_prefix}")
        self.vlm.prefill(input_ids, pixel_values, image_grid_thw)
        return S, int(self.vlm._next_pos)

    # ------------------------------------------------------------------ denoise
    def _denoise_loop(self, num_steps: int) -> None:
        cfg, K, sch = self.cfg, self.K, self.schedule(num_steps)
        n = cfg.suffix_rows
        for k in range(num_steps):
            K.gemm(self.x, sch["enc_w"], bias=sch["enc_b"][k], act="silu", out=self.enc)
            K.gemm(self.enc, sch["out_w_t"], bias=sch["out_b_t"], out=self.h[1:])
            self.h[0:1].copy_(self.state_emb)
            self.expert.forward(self.h, q_start=self.s_qstart, q_len=self.s_qlen, kv_len=self.s_kvlen, max_q_len=n,
                                max_kv_len=self.max_seq, pos=self.s_pos, cos=self.cos, sin=self.sin,
                                seq_of_tok=self.s_seq, cache_pos=self.s_cache_pos, page_table=self.cache.page_table,
                                mask=self.mask, mod=sch["film"][k], rows_per_mod=n)
            K.rmsnorm(self.h, self.final_norm_w, cfg.eps, out=self.hn)
            K.gemm(self.hn[1:], sch["out_w"], bias=sch["out_b"], residual=self.x, out=self.x)      # x <- x + dt * v

    @torch.no_grad()
    def denoise(self, prefix_len: int, p0: int, state: torch.Tensor, noise: torch.Tensor, num_steps: Optional[int] = None,
                *, use_graph: bool = True) -> torch.Tensor:
        cfg, dev = self.cfg, self.device
        num_steps = num_steps or cfg.num_steps
        n = cfg.suffix_rows
        self.cache.ensure(0, prefix_len + n)
        self.cache.sync_table()
        ar = torch.arange(n, dtype=torch.int32)
        self.s_pos.copy_((ar + p0).to(dev), non_blocking=True)
        self.s_cache_pos.copy_((ar + prefix_len).to(dev), non_blocking=True)
        self.s_kvlen.fill_(prefix_len + n)
        self.mask.copy_(suffix_mask(cfg, prefix_len, self.max_seq).to(torch.uint8).to(dev), non_blocking=True)
        st = F.linear(state.to(dev, torch.float32).reshape(1, -1), self.state_w, self.state_b)
        self.state_emb.copy_(st.to(self.dtype))
        self.x.zero_()
        self.x[:, :cfg.action_dim].copy_(noise.reshape(cfg.horizon, cfg.action_dim).to(dev, self.dtype))
        if not use_graph:
            self._denoise_loop(num_steps)
        else:
            gph = self._graphs.get(num_steps)
            if gph is None:
                snap = self.x.clone()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._denoise_loop(1)                          # warm-up: load kernels, set attributes
                torch.cuda.current_stream().wait_stream(s)
                self.schedule(num_steps)
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph, stream=s):
                    self._denoise_loop(num_steps)
                torch.cuda.synchronize()
                self.x.copy_(snap)
                self._graphs[num_steps] = gph
            gph.replay()
        return self.x[:, :cfg.action_dim]

    @torch.no_grad()
    def predict(self, input_ids, pixel_values, image_grid_thw, state, noise, num_steps: Optional[int] = None, *,
                use_graph: bool = True) -> torch.Tensor:
        S, p0 = self.prefill(input_ids, pixel_values, image_grid_thw)
        return self.denoise(S, p0, state, noise, num_steps, use_graph=use_graph)

    def check_status(self) -> None:
        self.vlm.text.check_status()
        self.expert.check_status()

    def close(self) -> None:
        self._graphs.clear()
        self.expert.close()
        self.vlm.close()
