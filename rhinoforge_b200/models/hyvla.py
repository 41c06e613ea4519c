"""Hy-Embodied VLA: a HunYuan-VL mixture-of-transformers prefix and a flow-matching action expert on one KV cache.

Two towers share the attention geometry (16 query heads, 4 KV heads of 128, 32 layers):

* the VLM tower reads the prompt.  It is a mixture of transformers: every layer holds TWO weight sets, and every row is
  routed to one of them by its modality (text rows -> the plain set, vision rows -> the ``_v`` twins; norms, q/k/v/o and
  the MLP all come in pairs, only the per-head ``query_layernorm`` / ``key_layernorm`` are shared).  Text and vision rows
  interleave finely (each image is 7 rows of 7 patches + 1 separator token), so routing is per row;
* the expert tower reads ``1 state + 50 action`` suffix rows per Euler step, attends to ``[prefix K/V | suffix]`` and runs
  through its ``_v`` weights only (a suffix row always counts as "vision"); its per-head q/k norm weights are the VLM
  layers', not its own.

Both towers apply RoPE *before* the per-head q/k RMSNorm, with the dynamic-NTK base
``theta * alpha^(hd / (hd - 2))`` and ``inv_freq`` rounded to bf16 as the checkpoint was trained.

Here the rows of the prefix are ordered ``[text rows | vision rows]`` once, so that each of a layer's projections and
norms is two launches over two contiguous row ranges (``NativeStack(..., twin_layer_weights=)``, ``twin_split``);
positions, cache rows and the attention mask are per row, so attention itself is indifferent to the order and K/V land
in the cache at the rows' original positions.  The vision path before that is the HYViT2 tower with the merger's first
projection as its per-token projector, then the merger's group pooling: the 14 x 14 tokens form 7 x 7 groups of 2 x 2
members, a two-layer predictor scores each member against the group mean, and the softmax-weighted member sum goes
through GELU and ``proj2``.  The expert's suffix encoder is folded per ``num_steps`` (input projection times the action
half of ``action_time_mlp_in`` as one matrix, the time half as a per-step bias) and the Euler loop replays from one
CUDA graph.

Reference behaviour: ``src/fused/rpu_hyvla_vlm_model.h:1-60`` (twin weights, row mask merge, shared q/k norms),
``src/fused/rpu_hyvla_expert_model.h:1-30`` (single tower, RoPE before head norm, VLM's norm weights),
``python/rpu_backend/adapters/hy_vla/weights.py:29-120,354-425,523-623`` (names, geometry, RoPE base, suffix encoder),
``adapters/hy_vla/runtime.py:374-397,546-606,607-820`` (prefix assembly, merger, pipeline).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

VIT_P = "model.dual_tower.vlm.model.visual.vision_tower."
MERGER_P = "model.dual_tower.vlm.model.visual.merger."
VLM_P = "model.dual_tower.vlm.model.language_model.model."
EXPERT_P = "model.dual_tower.expert.model."
LM_HEAD = "model.dual_tower.vlm.model.language_model.lm_head.weight"
HEAD_NAMES = ("state_proj", "action_in_proj", "action_time_mlp_in", "action_time_mlp_out", "action_out_proj")


@dataclass
class HyVlaConfig:
    layers: int = 32
    heads: int = 16
    kv_heads: int = 4
    head_dim: int = 128
    eps: float = 1e-5
    vlm_hidden: int = 2048
    vlm_inter: int = 6144
    expert_hidden: int = 1024
    expert_inter: int = 2048
    grid: int = 7                    # merged tokens per image side (the tower gives 2 * grid per side)
    vit_hidden: int = 1152
    n_action: int = 50
    action_dim: int = 32
    state_dim: int = 32
    num_steps: int = 10
    rope_theta: float = 10000.0
    rope_alpha: float = 1000.0
    vocab: int = 120818
    tok_bos: int = 120000
    tok_user: int = 120006
    tok_vision_start: int = 120684
    tok_vision_end: int = 120685
    tok_vision_split: int = 120689

    @property
    def suffix_len(self) -> int:
        return 1 + self.n_action

    @property
    def rope_base(self) -> float:
        return self.rope_theta * self.rope_alpha ** (self.head_dim / (self.head_dim - 2))


def tiny_hyvla_config(**kw) -> HyVlaConfig:
    base = dict(layers=3, heads=2, kv_heads=1, head_dim=64, vlm_hidden=128, vlm_inter=256, expert_hidden=64, expert_inter=128,
                grid=2, vit_hidden=96, n_action=6, action_dim=8, state_dim=8, num_steps=4, rope_alpha=10.0, vocab=64, tok_bos=60,
                tok_user=61, tok_vision_start=62, tok_vision_end=63, tok_vision_split=59)
    base.update(kw)
    return HyVlaConfig(**base)


def hyvla_shapes(cfg: HyVlaConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """(checkpoint name, shape, kind) of the two decoder towers, the merger and the action head (the vision tower's own
    tensors are the HYViT2 encoder's)."""
    hd, Hq, Hkv = cfg.head_dim, cfg.heads, cfg.kv_heads
    for tower, H, I, sets in ((VLM_P, cfg.vlm_hidden, cfg.vlm_inter, ("", "_v")), (EXPERT_P, cfg.expert_hidden, cfg.expert_inter, ("_v",))):
        for i in range(cfg.layers):
            b = f"{tower}layers.{i}."
            for s in sets:
                yield b + f"self_attn.q_proj{s}.weight", (Hq * hd, H), "matrix"
                yield b + f"self_attn.k_proj{s}.weight", (Hkv * hd, H), "matrix"
                yield b + f"self_attn.v_proj{s}.weight", (Hkv * hd, H), "matrix"
                yield b + f"self_attn.o_proj{s}.weight", (H, Hq * hd), "matrix"
                yield b + f"mlp{s}.gate_proj.weight", (I, H), "matrix"
                yield b + f"mlp{s}.up_proj.weight", (I, H), "matrix"
                yield b + f"mlp{s}.down_proj.weight", (H, I), "matrix"
                yield b + f"input_layernorm{s}.weight", (H,), "norm"
                yield b + f"post_attention_layernorm{s}.weight", (H,), "norm"
            if tower == VLM_P:
                yield b + "self_attn.query_layernorm.weight", (hd,), "norm"
                yield b + "self_attn.key_layernorm.weight", (hd,), "norm"
        yield tower + "norm.weight", (H,), "norm"
    D, V = cfg.vlm_hidden, cfg.vit_hidden
    yield MERGER_P + "proj1.weight", (D, V), "matrix"
    yield MERGER_P + "proj1.bias", (D,), "bias"
    yield MERGER_P + "pooler.predictor.0.weight", (D, 2 * D), "matrix"
    yield MERGER_P + "pooler.predictor.0.bias", (D,), "bias"
    yield MERGER_P + "pooler.predictor.2.weight", (D, D), "matrix"
    yield MERGER_P + "pooler.predictor.2.bias", (D,), "bias"
    yield MERGER_P + "proj2.weight", (D, D), "matrix"
    yield MERGER_P + "proj2.bias", (D,), "bias"
    yield LM_HEAD, (cfg.vocab, D), "embed"
    E = cfg.expert_hidden
    yield "model.state_proj.weight", (E, cfg.state_dim), "matrix"
    yield "model.state_proj.bias", (E,), "bias"
    yield "model.action_in_proj.weight", (E, cfg.action_dim), "matrix"
    yield "model.action_in_proj.bias", (E,), "bias"
    yield "model.action_time_mlp_in.weight", (E, 2 * E), "matrix"
    yield "model.action_time_mlp_in.bias", (E,), "bias"
    yield "model.action_time_mlp_out.weight", (E, E), "matrix"
    yield "model.action_time_mlp_out.bias", (E,), "bias"
    yield "model.action_out_proj.weight", (cfg.action_dim, E), "matrix"
    yield "model.action_out_proj.bias", (cfg.action_dim,), "bias"


def random_hyvla_state_dict(cfg: HyVlaConfig, *, seed: int = 0, std: float = 0.06, dtype=torch.float32,
                            device="cpu") -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in hyvla_shapes(cfg):
        r = torch.randn(shape, generator=g)
        sd[name] = {"matrix": r * std, "embed": r * 0.5, "norm": 1.0 + 0.05 * r, "bias": 0.03 * r}[kind].to(device, dtype)
    return sd


# ----------------------------------------------------------------------------- shared pieces
def rope_tables(cfg: HyVlaConfig, max_pos: int, *, bf16_inv_freq: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """``cos, sin [max_pos, head_dim / 2]`` fp32 on the dynamic-NTK base; ``inv_freq`` rounded to bf16 first."""
    hd = cfg.head_dim
    inv = 1.0 / (cfg.rope_base ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    if bf16_inv_freq:
        inv = inv.float().to(torch.bfloat16).double()
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv)
    return ang.cos().float(), ang.sin().float()


def step_times(num_steps: int) -> List[float]:
    return [1.0 - k / num_steps for k in range(num_steps)]


def time_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    """``[n] -> [n, dim]`` fp32: sin | cos over ``dim / 2`` periods interpolated geometrically from 4e-3 to 4."""
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64)
    period = 4e-3 * (4.0 / 4e-3) ** frac
    ang = (2.0 * math.pi / period)[None, :] * t.double()[:, None]
    return torch.cat((ang.sin(), ang.cos()), 1).float()


def folded_suffix_encoder(sd: Dict[str, torch.Tensor], cfg: HyVlaConfig, num_steps: int):
    """``(W [E, action_dim], step_bias [num_steps, E])`` fp32 with ``silu(x @ W.T + step_bias[k])`` equal to
    ``silu(mlp_in(cat(action_in(x), time_embedding(t_k))))``."""
    E = cfg.expert_hidden
    w1, b1 = sd["model.action_time_mlp_in.weight"].float(), sd["model.action_time_mlp_in.bias"].float()
    wa, wt = w1[:, :E], w1[:, E:]
    wi, bi = sd["model.action_in_proj.weight"].float(), sd["model.action_in_proj.bias"].float()
    te = time_embedding(torch.tensor(step_times(num_steps)), E).to(w1.device)
    return (wa @ wi).contiguous(), (F.linear(te, wt, b1) + F.linear(bi, wa)[None]).contiguous()


def merger_pool(sd: Dict[str, torch.Tensor], cfg: HyVlaConfig, proj1_out: torch.Tensor) -> torch.Tensor:
    """The merger behind ``proj1``: ``[B, (2 grid)^2, D]`` tokens in raster order -> ``[B, grid^2, D]``: every 2 x 2 group's
    members are scored (two-layer predictor on ``[member | group mean]``), soft-maxed over the group and summed with those
    weights, then GELU and ``proj2``."""
    g, D = cfg.grid, proj1_out.shape[-1]
    B = proj1_out.shape[0]
    nxc = proj1_out.float().reshape(B, g, 2, g, 2, D).permute(0, 1, 3, 2, 4, 5).reshape(B, g, g, 4, D)
    pooled = nxc.mean(-2, keepdim=True).expand(-1, -1, -1, 4, -1)
    p = lambda n: sd[MERGER_P + n].float().to(proj1_out.device)
    sc = F.linear(torch.cat((nxc, pooled), -1), p("pooler.predictor.0.weight"), p("pooler.predictor.0.bias"))
    sc = F.linear(F.gelu(sc), p("pooler.predictor.2.weight"), p("pooler.predictor.2.bias"))
    out = (nxc * torch.softmax(sc, dim=-2)).sum(-2)
    return F.linear(F.gelu(out), p("proj2.weight"), p("proj2.bias")).reshape(B, g * g, D)


def assemble_prefix(cfg: HyVlaConfig, tok_emb: torch.Tensor, img_embs: Sequence[torch.Tensor], lang_tokens: torch.Tensor):
    """``(rows [S, D], is_vision [S])``: ``[bos, user] + per image (start + grid rows of (grid patches + 1 split) + end) +
    language tokens``; only the patch rows are vision rows."""
    g, D = cfg.grid, tok_emb.shape[1]
    t = lambda i: tok_emb[i][None]
    parts, vis = [t(cfg.tok_bos), t(cfg.tok_user)], [False, False]
    for ie in img_embs:
        parts.append(t(cfg.tok_vision_start))
        vis.append(False)
        grid = torch.cat((ie.reshape(g, g, D).to(tok_emb.dtype), tok_emb[cfg.tok_vision_split][None, None].expand(g, 1, D)), 1)
        parts.append(grid.reshape(g * (g + 1), D))
        vis += ([True] * g + [False]) * g
        parts.append(t(cfg.tok_vision_end))
        vis.append(False)
    parts.append(tok_emb[lang_tokens.long()])
    vis += [False] * int(lang_tokens.numel())
    return torch.cat(parts, 0), torch.tensor(vis)


def _tower_layers(sd: Dict[str, torch.Tensor], cfg: HyVlaConfig, tower: str, s: str) -> List[Dict[str, torch.Tensor]]:
    """Per-layer weight sets of one tower and weight-set suffix in the native stack's field names; the per-head q/k norm
    weights are always the VLM layers'."""
    out = []
    for i in range(cfg.layers):
        b = f"{tower}layers.{i}."
        out.append(dict(
            norm1_w=sd[b + f"input_layernorm{s}.weight"], norm2_w=sd[b + f"post_attention_layernorm{s}.weight"],
            wqkv=torch.cat([sd[b + f"self_attn.{x}_proj{s}.weight"] for x in "qkv"], 0), wo=sd[b + f"self_attn.o_proj{s}.weight"],
            q_norm_w=sd[f"{VLM_P}layers.{i}.self_attn.query_layernorm.weight"],
            k_norm_w=sd[f"{VLM_P}layers.{i}.self_attn.key_layernorm.weight"],
            w_up=torch.cat((sd[b + f"mlp{s}.gate_proj.weight"], sd[b + f"mlp{s}.up_proj.weight"]), 0),
            w_down=sd[b + f"mlp{s}.down_proj.weight"]))
    return out


# ----------------------------------------------------------------------------- fp32 oracle
class TorchHyVla:
    """Plain PyTorch statement of both towers (row-by-row weight selection, no reordering, no folds)."""

    def __init__(self, cfg: HyVlaConfig, sd: Dict[str, torch.Tensor], *, dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.sd = {k: v.to(self.device, dtype) for k, v in sd.items()}
        self.cos, self.sin = (t.to(self.device) for t in rope_tables(cfg, 4096))

    def _rms(self, t, w):
        tf = t.float()
        return (tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * w.float()).to(self.dtype)

    def _rope(self, t, pos):      # t [n, heads, hd]
        cos = torch.cat((self.cos[pos], self.cos[pos]), -1)[:, None]
        sin = torch.cat((self.sin[pos], self.sin[pos]), -1)[:, None]
        h = t.shape[-1] // 2
        return (t.float() * cos + torch.cat((-t[..., h:], t[..., :h]), -1).float() * sin).to(t.dtype)

    def _layer(self, tower, i, h, pick, pos, mask, past):
        """``pick(name_without_suffix) -> per-row weights``: returns a function applying the right set per row."""
        cfg, sd = self.cfg, self.sd
        hd, G = cfg.head_dim, cfg.heads // cfg.kv_heads
        n = h.shape[0]
        b = f"{tower}layers.{i}."
        y = pick(lambda s: self._rms(h, sd[b + f"input_layernorm{s}.weight"]))
        q = pick(lambda s: F.linear(y, sd[b + f"self_attn.q_proj{s}.weight"])).view(n, cfg.heads, hd)
        k = pick(lambda s: F.linear(y, sd[b + f"self_attn.k_proj{s}.weight"])).view(n, cfg.kv_heads, hd)
        v = pick(lambda s: F.linear(y, sd[b + f"self_attn.v_proj{s}.weight"])).view(n, cfg.kv_heads, hd)
        qn, kn = sd[f"{VLM_P}layers.{i}.self_attn.query_layernorm.weight"], sd[f"{VLM_P}layers.{i}.self_attn.key_layernorm.weight"]
        q, k = self._rms(self._rope(q, pos), qn), self._rms(self._rope(k, pos), kn)       # RoPE first, then the head norm
        if past is not None:
            k, v = torch.cat((past[0], k), 0), torch.cat((past[1], v), 0)
        kk, vv = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
        s_ = torch.einsum("qhd,khd->hqk", q.float(), kk.float()) / math.sqrt(hd)
        s_ = s_.masked_fill(~mask[None], float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s_, -1), vv.float()).to(self.dtype).reshape(n, -1)
        h = h + pick(lambda s: F.linear(o, sd[b + f"self_attn.o_proj{s}.weight"]))
        y = pick(lambda s: self._rms(h, sd[b + f"post_attention_layernorm{s}.weight"]))
        m = pick(lambda s: F.linear(F.silu(F.linear(y, sd[b + f"mlp{s}.gate_proj.weight"])) * F.linear(y, sd[b + f"mlp{s}.up_proj.weight"]),
                                    sd[b + f"mlp{s}.down_proj.weight"]))
        return h + m, (k, v)

    @torch.no_grad()
    def prefill(self, rows: torch.Tensor, pos: torch.Tensor, mask: torch.Tensor, is_vision: torch.Tensor):
        """MoT prefill: returns per-layer ``(K, V) [S, kv_heads, hd]`` (rotated, head-normed keys)."""
        h = rows.to(self.device, self.dtype)
        vis = is_vision.to(self.device).bool()[:, None]
        mask = mask.to(self.device).bool() | torch.eye(h.shape[0], dtype=torch.bool, device=self.device)

        def pick(f):
            a, b = f(""), f("_v")
            return torch.where(vis.view(-1, *([1] * (a.dim() - 1))), b, a)
        kv = []
        for i in range(self.cfg.layers):
            h, kvi = self._layer(VLM_P, i, h, pick, pos.to(self.device).long(), mask, None)
            kv.append(kvi)
        return kv

    @torch.no_grad()
    def sample_actions(self, kv, suffix_pos: torch.Tensor, denoise_mask: torch.Tensor, state: torch.Tensor, noise: torch.Tensor,
                       num_steps: Optional[int] = None) -> torch.Tensor:
        cfg, sd = self.cfg, self.sd
        num_steps = num_steps or cfg.num_steps
        E = cfg.expert_hidden
        x = noise.reshape(cfg.n_action, cfg.action_dim).to(self.device, self.dtype)
        st = F.linear(state.to(self.device, self.dtype).reshape(1, -1), sd["model.state_proj.weight"], sd["model.state_proj.bias"])
        mask = denoise_mask.to(self.device).bool()
        pos = suffix_pos.to(self.device).long()
        dt = -1.0 / num_steps
        for t in step_times(num_steps):
            te = time_embedding(torch.tensor([t]), E).to(self.device, self.dtype).expand(cfg.n_action, -1)
            a = F.linear(x, sd["model.action_in_proj.weight"], sd["model.action_in_proj.bias"])
            a = F.silu(F.linear(torch.cat((a, te), -1), sd["model.action_time_mlp_in.weight"], sd["model.action_time_mlp_in.bias"]))
            a = F.linear(a, sd["model.action_time_mlp_out.weight"], sd["model.action_time_mlp_out.bias"])
            h = torch.cat((st, a), 0)
            for i in range(cfg.layers):
                h, _ = self._layer(EXPERT_P, i, h, lambda f: f("_v"), pos, mask, kv[i])
            hn = self._rms(h, sd[EXPERT_P + "norm.weight"])
            x = x + dt * F.linear(hn[-cfg.n_action:], sd["model.action_out_proj.weight"], sd["model.action_out_proj.bias"])
        return x


# ----------------------------------------------------------------------------- device engine
class HyVlaEngine:
    """Both towers on the accelerator.  ``vision`` (optional) is a callable ``images -> [n_img, (2 grid)^2, vlm_hidden]``
    (the HYViT2 tower with ``proj1`` as its projector); without it :meth:`prefill` takes ready prefix rows."""

    def __init__(self, cfg: HyVlaConfig, sd: Dict[str, torch.Tensor], *, max_prefix: int = 256, device="cuda",
                 dtype=torch.float16, vision=None):
        from ..ops import kernels as K
        from ..runtime.kv_cache import PagedKV
        from ..runtime.stack import NativeStack, StackSpec
        self.K, self.cfg, self.device, self.dtype, self.vision = K, cfg, torch.device(device), dtype, vision
        dev, L = self.device, cfg.suffix_len
        self.max_prefix = max_prefix
        self.max_seq = (max_prefix + L + 15) // 16 * 16
        self.cache = PagedKV(cfg.layers, 1, self.max_seq, cfg.kv_heads, cfg.head_dim, device=device, dtype=dtype)
        self.cache.reserve_all()
        common = dict(layers=cfg.layers, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, norm="rms", mlp="swiglu",
                      eps=cfg.eps, qk_norm=True, rope_before_norm=True, rot_dim=cfg.head_dim, paged_kv=True, causal=False,
                      max_seqs=1)
        self.vlm = NativeStack(StackSpec(hidden=cfg.vlm_hidden, inter=cfg.vlm_inter, max_tokens=(max_prefix + 15) // 16 * 16, **common),
                               _tower_layers(sd, cfg, VLM_P, ""), device=device, dtype=dtype, kv_cache=self.cache,
                               twin_layer_weights=_tower_layers(sd, cfg, VLM_P, "_v"))
        self.expert = NativeStack(StackSpec(hidden=cfg.expert_hidden, inter=cfg.expert_inter, max_tokens=(L + 15) // 16 * 16, **common),
                                  _tower_layers(sd, cfg, EXPERT_P, "_v"), device=device, dtype=dtype, kv_cache=self.cache,
                                  final_norm_w=sd[EXPERT_P + "norm.weight"])
        cos, sin = rope_tables(cfg, self.max_seq + 4096)
        self.cos, self.sin = cos.to(dev).contiguous(), sin.to(dev).contiguous()
        self.tok_emb = sd[LM_HEAD].to(dev, dtype)
        keep = [n for n, _, _ in hyvla_shapes(cfg) if n.startswith(("model.state_proj", "model.action_", MERGER_P))]
        self._small = {k: sd[k].to(dev, torch.float32) for k in keep}
        self.ad_pad = (cfg.action_dim + 7) // 8 * 8
        self._schedules: Dict[int, dict] = {}
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        i32 = dict(dtype=torch.int32, device=dev)
        E = cfg.expert_hidden
        self.x = torch.zeros(cfg.n_action, self.ad_pad, dtype=dtype, device=dev)
        self.h = torch.zeros(L, E, dtype=dtype, device=dev)
        self.hn = torch.zeros(L, E, dtype=dtype, device=dev)
        self.enc = torch.zeros(cfg.n_action, E, dtype=dtype, device=dev)
        self.state_emb = torch.zeros(1, E, dtype=dtype, device=dev)
        self.s_pos = torch.zeros(L, **i32)
        self.s_cache_pos = torch.zeros(L, **i32)
        self.s_seq = torch.zeros(L, **i32)
        self.s_qstart = torch.zeros(1, **i32)
        self.s_qlen = torch.full((1,), L, **i32)
        self.s_kvlen = torch.zeros(1, **i32)
        self.mask = torch.zeros(L, (self.max_seq + 127) // 128 * 128, dtype=torch.uint8, device=dev)[:, :self.max_seq]   # pitch: whole 128-key blocks
        self.p_hidden = torch.zeros(self.vlm.spec.max_tokens, cfg.vlm_hidden, dtype=dtype, device=dev)
        self.prefix_len = 0

    # ------------------------------------------------------------------ vision + prefix rows
    @torch.no_grad()
    def embed_images(self, images: torch.Tensor) -> torch.Tensor:
        """``[n_img, 3, H, W]`` -> ``[n_img, grid^2, vlm_hidden]`` (tower with ``proj1``, then the merger's group pooling)."""
        if self.vision is None:
            raise ValueError("this engine was built without a vision tower")
        return merger_pool(self._small, self.cfg, self.vision(images)).to(self.dtype)

    def build_prefix(self, img_embs: Sequence[torch.Tensor], lang_tokens: torch.Tensor):
        return assemble_prefix(self.cfg, self.tok_emb, [e.to(self.device) for e in img_embs], lang_tokens.to(self.device))

    # ------------------------------------------------------------------ MoT prefill
    @torch.no_grad()
    def prefill(self, rows: torch.Tensor, pos: torch.Tensor, mask: torch.Tensor, is_vision: torch.Tensor) -> int:
        """Run the prefix (``rows [S, vlm_hidden]``, positions ``[S]``, boolean mask ``[S, S]``, modality flags ``[S]``)
        through the twin-weight tower; K/V of every layer land in cache rows ``[0, S)`` in the prefix's own order."""
        cfg, dev = self.cfg, self.device
        S = int(rows.shape[0])
        if S > self.max_prefix:
            raise ValueError(f"prefix of {S} rows exceeds max_prefix {self.max_prefix}")
        vis = is_vision.flatten().bool().cpu()
        perm = torch.cat(((~vis).nonzero().flatten(), vis.nonzero().flatten()))          # text rows, then vision rows
        split = int((~vis).sum())
        if split == 0 or split == S:
            raise ValueError("the mixture-of-transformers prefill needs rows of both modalities")
        m = mask.bool().cpu() | torch.eye(S, dtype=torch.bool)                           # a padded row still sees itself
        h = self.p_hidden[:S]
        h.copy_(rows.to(dev, self.dtype)[perm.to(dev)])
        i32 = lambda t: t.to(torch.int32).to(dev)
        kv_len = torch.tensor([S], dtype=torch.int32, device=dev)
        self.cache.ensure(0, S + cfg.suffix_len)
        self.cache.sync_table()
        self.vlm.forward(h, q_start=torch.zeros(1, dtype=torch.int32, device=dev), q_len=kv_len, kv_len=kv_len, max_q_len=S,
                         max_kv_len=S, pos=i32(pos.flatten().cpu()[perm]), cos=self.cos, sin=self.sin,
                         seq_of_tok=torch.zeros(S, dtype=torch.int32, device=dev), cache_pos=i32(perm),
                         page_table=self.cache.page_table, mask=m[perm].to(torch.uint8).to(dev).contiguous(), twin_split=split)
        self.prefix_len = S
        return S

    # ------------------------------------------------------------------ denoise
    def schedule(self, num_steps: int) -> dict:
        hit = self._schedules.get(num_steps)
        if hit is not None:
            return hit
        cfg, sd = self.cfg, self._small
        wf, sb = folded_suffix_encoder(sd, cfg, num_steps)
        dt = -1.0 / num_steps
        pad = lambda w, rows, cols: F.pad(w, (0, cols - w.shape[1], 0, rows - w.shape[0]))
        hit = dict(enc_w=pad(wf, cfg.expert_hidden, self.ad_pad).to(self.dtype).contiguous(), enc_b=sb.to(self.dtype).contiguous(),
                   mo_w=sd["model.action_time_mlp_out.weight"].to(self.dtype).contiguous(),
                   mo_b=sd["model.action_time_mlp_out.bias"].to(self.dtype).contiguous(),
                   out_w=pad(sd["model.action_out_proj.weight"] * dt, self.ad_pad, cfg.expert_hidden).to(self.dtype).contiguous(),
                   out_b=F.pad(sd["model.action_out_proj.bias"] * dt, (0, self.ad_pad - cfg.action_dim)).to(self.dtype).contiguous())
        self._schedules[num_steps] = hit
        return hit

    def _denoise_loop(self, num_steps: int) -> None:
        cfg, K, sch = self.cfg, self.K, self.schedule(num_steps)
        L = cfg.suffix_len
        for k in range(num_steps):
            K.gemm(self.x, sch["enc_w"], bias=sch["enc_b"][k], act="silu", out=self.enc)
            K.gemm(self.enc, sch["mo_w"], bias=sch["mo_b"], out=self.h[1:])
            self.h[0:1].copy_(self.state_emb)
            self.expert.forward(self.h, q_start=self.s_qstart, q_len=self.s_qlen, kv_len=self.s_kvlen, max_q_len=L,
                                max_kv_len=self.max_seq, pos=self.s_pos, cos=self.cos, sin=self.sin, seq_of_tok=self.s_seq,
                                cache_pos=self.s_cache_pos, page_table=self.cache.page_table, mask=self.mask)
            self.expert.final_norm(self.h, out=self.hn)
            K.gemm(self.hn[1:], sch["out_w"], bias=sch["out_b"], residual=self.x, out=self.x)     # x <- x + dt * v

    @torch.no_grad()
    def denoise(self, suffix_pos: torch.Tensor, denoise_mask: torch.Tensor, state: torch.Tensor, noise: torch.Tensor,
                num_steps: Optional[int] = None, *, use_graph: bool = True) -> torch.Tensor:
        """Euler loop over the current prefix.  ``suffix_pos [suffix_len]`` are the suffix rows' positions (they continue
        from the prefix's VALID length); ``denoise_mask [suffix_len, prefix_len + suffix_len]`` says what each suffix row
        sees.  Returns ``[n_action, action_dim]`` in a buffer the next call overwrites."""
        cfg, dev = self.cfg, self.device
        num_steps = num_steps or cfg.num_steps
        L, S = cfg.suffix_len, self.prefix_len
        if tuple(denoise_mask.shape) != (L, S + L):
            raise ValueError(f"denoise_mask must be {(L, S + L)}, got {tuple(denoise_mask.shape)}")
        self.s_pos.copy_(suffix_pos.flatten().to(torch.int32).to(dev))
        self.s_cache_pos.copy_((torch.arange(L, dtype=torch.int32) + S).to(dev))
        self.s_kvlen.fill_(S + L)
        m = torch.zeros(L, self.max_seq, dtype=torch.bool)
        m[:, :S + L] = denoise_mask.bool().cpu()
        self.mask.copy_(m.to(torch.uint8).to(dev))
        st = F.linear(state.to(dev, torch.float32).reshape(1, -1), self._small["model.state_proj.weight"],
                      self._small["model.state_proj.bias"])
        self.state_emb.copy_(st.to(self.dtype))
        self.x.zero_()
        self.x[:, :cfg.action_dim].copy_(noise.reshape(cfg.n_action, cfg.action_dim).to(dev, self.dtype))
        if not use_graph:
            self._denoise_loop(num_steps)
        else:
            gph = self._graphs.get(num_steps)
            if gph is None:
                snap = self.x.clone()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._denoise_loop(1)                              # warm-up: load kernels, set attributes
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

    def check_status(self) -> None:
        self.vlm.check_status()
        self.expert.check_status()

    def close(self) -> None:
        self._graphs.clear()
        self.vlm.close()
        self.expert.close()
        self.cache.close()


__all__ = ["HyVlaConfig", "HyVlaEngine", "TorchHyVla", "tiny_hyvla_config", "hyvla_shapes", "random_hyvla_state_dict",
           "rope_tables", "step_times", "time_embedding", "folded_suffix_encoder", "merger_pool", "assemble_prefix",
           "VIT_P", "MERGER_P", "VLM_P", "EXPERT_P", "LM_HEAD"]
