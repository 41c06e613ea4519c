"""GR00T-N1.7 action head: the VL encoder (LayerNorm + 4 bidirectional transformer blocks over the backbone's hidden
states) and the flow-matching DiT (32 blocks that alternate cross-attention over the vision-language tokens with
self-attention over 1 state + 40 action tokens), with per-embodiment encoders / decoder and a 4-step Euler loop.

Per Euler step ``s`` (``t_s = int(s / steps * 1000)``, ``dt = 1 / steps``)::

    cond   = silu(timestep_embedder(t_s))                                  # [H]; a table
    a_emb  = W1 x ; af = W3 silu(W2 [a_emb | sincos(t_s)]) + pos           # action encoder, per embodiment
    h      = [state_feat ; af]                                             # 41 rows
    block i: h += attn(LN(h) (1 + scale_i) + shift_i) ; h += FF(LN(h))     # [scale_i | shift_i] = A_i cond + a_i
             even i: keys / values are projections of the VL tokens; i % 4 == 0 sees the text tokens, i % 4 == 2 the
             image tokens;  odd i: self-attention over the 41 rows (no mask)
    out    = P2 (LN(h) (1 + scale_o) + shift_o) ; pred = D2 relu(D1 out)   # [shift_o | scale_o] = P1 cond + p1
    x     += dt * pred[1:]

Everything that does not depend on ``x`` is computed once: the modulation rows of every (step, block) and of the output
norm are tables built with the engine; the sinusoidal half of the action encoder's second layer sits pre-filled in the
K-concatenated input buffer of every step; the VL tokens are re-ordered ``[text | image]`` once per call so that each
cross block attends a contiguous row range without a mask, and go through all sixteen K/V projections before the loop.
Heads of 48 run on the 64-wide attention kernels with zero-padded head columns.  The loop (7 launches per block)
replays from one CUDA graph per VL length.

Reference behaviour: ``src/fused/rpu_gr00t_dit_model.cpp:1-21,1060-1210,1240-1325`` (block recipes, encoders, output
head, Euler update), ``src/fused/rpu_gr00t_vl_encoder_model.cpp:1-20`` (VL encoder),
``python/rpu_backend/adapters/gr00t/runtime.py:984-1015,1061-1227`` (masks, tensor names, baked tables).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterator, Optional, Tuple

import torch
import torch.nn.functional as F

AP = "action_head."


@dataclass
class Gr00tConfig:
    hidden: int = 1536              # DiT width
    heads: int = 32
    head_dim: int = 48
    ff: int = 6144
    layers: int = 32
    vl_dim: int = 2048              # backbone / VL encoder width
    vl_heads: int = 32
    vl_head_dim: int = 64
    vl_ff: int = 8192
    vl_layers: int = 4
    horizon: int = 40
    action_dim: int = 132
    state_dim: int = 132
    enc_mid: int = 1024             # state-encoder hidden width
    model_out: int = 1024           # DiT output width (input of the action decoder)
    dec_mid: int = 1024
    time_embed: int = 256           # sinusoidal width of the timestep embedder
    max_pos: int = 1024
    embodiments: int = 32
    steps: int = 4
    buckets: int = 1000
    eps: float = 1e-5
    eps_out: float = 1e-6

    def bucket(self, s: int) -> int:
        return int((s / self.steps) * self.buckets)


def tiny_gr00t_config(**kw) -> Gr00tConfig:
    base = dict(hidden=96, heads=2, head_dim=48, ff=192, layers=4, vl_dim=128, vl_heads=2, vl_head_dim=64, vl_ff=256, vl_layers=2,
                horizon=6, action_dim=12, state_dim=12, enc_mid=64, model_out=64, dec_mid=64, time_embed=32, max_pos=16,
                embodiments=3, steps=3)
    base.update(kw)
    return Gr00tConfig(**base)


def _block_shapes(p: str, dim: int, kv_in: int, ff: int, *, ada: bool):
    yield p + "attn1.to_q.weight", (dim, dim), "matrix"
    yield p + "attn1.to_k.weight", (dim, kv_in), "matrix"
    yield p + "attn1.to_v.weight", (dim, kv_in), "matrix"
    yield p + "attn1.to_out.0.weight", (dim, dim), "matrix"
    for n in ("to_q", "to_k", "to_v", "to_out.0"):
        yield p + f"attn1.{n}.bias", (dim,), "bias"
    yield p + "ff.net.0.proj.weight", (ff, dim), "matrix"
    yield p + "ff.net.0.proj.bias", (ff,), "bias"
    yield p + "ff.net.2.weight", (dim, ff), "matrix"
    yield p + "ff.net.2.bias", (dim,), "bias"
    if ada:
        yield p + "norm1.linear.weight", (2 * dim, dim), "small"
        yield p + "norm1.linear.bias", (2 * dim,), "bias"
    else:
        for n in ("norm1", "norm3"):
            yield p + n + ".weight", (dim,), "norm"
            yield p + n + ".bias", (dim,), "bias"


def gr00t_shapes(cfg: Gr00tConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    H, E = cfg.hidden, cfg.embodiments
    yield AP + "vlln.weight", (cfg.vl_dim,), "norm"
    yield AP + "vlln.bias", (cfg.vl_dim,), "bias"
    for i in range(cfg.vl_layers):
        yield from _block_shapes(f"{AP}vl_self_attention.transformer_blocks.{i}.", cfg.vl_dim, cfg.vl_dim, cfg.vl_ff, ada=False)
    for i in range(cfg.layers):
        yield from _block_shapes(f"{AP}model.transformer_blocks.{i}.", H, cfg.vl_dim if i % 2 == 0 else H, cfg.ff, ada=True)
    te = AP + "model.timestep_encoder.timestep_embedder."
    yield te + "linear_1.weight", (H, cfg.time_embed), "matrix"
    yield te + "linear_1.bias", (H,), "bias"
    yield te + "linear_2.weight", (H, H), "matrix"
    yield te + "linear_2.bias", (H,), "bias"
    yield AP + "model.proj_out_1.weight", (2 * H, H), "small"
    yield AP + "model.proj_out_1.bias", (2 * H,), "bias"
    yield AP + "model.proj_out_2.weight", (cfg.model_out, H), "matrix"
    yield AP + "model.proj_out_2.bias", (cfg.model_out,), "bias"
    yield AP + "position_embedding.weight", (cfg.max_pos, H), "embed"
    for name, i, o in (("state_encoder.layer1", cfg.state_dim, cfg.enc_mid), ("state_encoder.layer2", cfg.enc_mid, H),
                       ("action_encoder.W1", cfg.action_dim, H), ("action_encoder.W2", 2 * H, H), ("action_encoder.W3", H, H),
                       ("action_decoder.layer1", cfg.model_out, cfg.dec_mid), ("action_decoder.layer2", cfg.dec_mid, cfg.action_dim)):
        yield AP + name + ".W", (E, i, o), "matrix"          # per-embodiment banks, stored [in, out]
        yield AP + name + ".b", (E, o), "bias"


def random_gr00t_state_dict(cfg: Gr00tConfig, *, seed: int = 0, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in gr00t_shapes(cfg):
        r = torch.randn(shape, generator=g)
        fan_in = shape[-2] if name.endswith(".W") else shape[-1]
        sd[name] = {"matrix": r / math.sqrt(fan_in), "small": r * 0.3 / math.sqrt(fan_in), "embed": r * 0.1,
                    "norm": 1.0 + 0.05 * r, "bias": 0.03 * r}[kind].to(dtype)
    return sd


def check_state_dict(cfg: Gr00tConfig, get) -> None:
    """``get(name)`` returns a tensor or raises ``KeyError``; every tensor of the profile must have its shape."""
    bad = []
    for name, shape, _ in gr00t_shapes(cfg):
        try:
            t = get(name)
        except KeyError:
            bad.append(f"{name}: missing")
            continue
        if tuple(t.shape) != shape:
            bad.append(f"{name}: {tuple(t.shape)}, expected {shape}")
    if bad:
        raise ValueError(f"GR00T action head does not fit the profile ({len(bad)} tensors): " + "; ".join(bad[:6]))


# ----------------------------------------------------------------------------- tables
def timestep_cond(get, cfg: Gr00tConfig, bucket: int) -> torch.Tensor:
    """``silu(timestep_embedder(bucket))`` ``[H]`` fp32: cos-first sinusoid, two linears with a SiLU between."""
    half = cfg.time_embed // 2
    te = AP + "model.timestep_encoder.timestep_embedder."
    w1 = get(te + "linear_1.weight").float()
    f = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=w1.device) / (half - 1))
    a = float(bucket) * f
    e = torch.cat((a.cos(), a.sin()))[None]
    h = F.silu(F.linear(e, w1, get(te + "linear_1.bias").float()))
    return F.silu(F.linear(h, get(te + "linear_2.weight").float(), get(te + "linear_2.bias").float()))[0]


def action_time_encoding(cfg: Gr00tConfig, bucket: int) -> torch.Tensor:
    """``[H]`` fp32 ``[sin | cos]`` of the action encoder (the same row for every action token)."""
    half = cfg.hidden // 2
    f = torch.exp(-torch.arange(half, dtype=torch.float32) * (math.log(10000.0) / half))
    a = float(bucket) * f
    return torch.cat((a.sin(), a.cos()))


def subset_order(image_mask: torch.Tensor, valid_mask: torch.Tensor):
    """Row order ``[text | image]`` of the valid VL tokens and the two counts."""
    im, ok = image_mask.reshape(-1).bool().cpu(), valid_mask.reshape(-1).bool().cpu()
    text, image = ((~im) & ok).nonzero().flatten(), (im & ok).nonzero().flatten()
    return torch.cat((text, image)), int(text.numel()), int(image.numel())


# ----------------------------------------------------------------------------- fp32 oracle
class TorchGr00t:
    def __init__(self, cfg: Gr00tConfig, sd: Dict[str, torch.Tensor], embodiment: int = 0, device="cpu"):
        self.cfg, self.emb, self.device = cfg, embodiment, torch.device(device)
        self.sd = {k: v.float().to(self.device) for k, v in sd.items()}

    def _attn(self, q, k, v, heads, hd):
        q, k, v = (t.reshape(t.shape[0], heads, hd).transpose(0, 1) for t in (q, k, v))
        return F.scaled_dot_product_attention(q, k, v).transpose(0, 1).reshape(q.shape[1], heads * hd)

    def _lin(self, x, name):
        return F.linear(x, self.sd[name + ".weight"], self.sd[name + ".bias"])

    def _cat(self, x, name):
        return x @ self.sd[AP + name + ".W"][self.emb] + self.sd[AP + name + ".b"][self.emb]

    @torch.no_grad()
    def vl_encode(self, hidden: torch.Tensor) -> torch.Tensor:
        cfg, sd = self.cfg, self.sd
        x = F.layer_norm(hidden.float().to(self.device), (cfg.vl_dim,), sd[AP + "vlln.weight"], sd[AP + "vlln.bias"], cfg.eps)
        for i in range(cfg.vl_layers):
            p = f"{AP}vl_self_attention.transformer_blocks.{i}."
            n = F.layer_norm(x, (cfg.vl_dim,), sd[p + "norm1.weight"], sd[p + "norm1.bias"], cfg.eps)
            a = self._attn(self._lin(n, p + "attn1.to_q"), self._lin(n, p + "attn1.to_k"), self._lin(n, p + "attn1.to_v"),
                           cfg.vl_heads, cfg.vl_head_dim)
            x = x + self._lin(a, p + "attn1.to_out.0")
            n = F.layer_norm(x, (cfg.vl_dim,), sd[p + "norm3.weight"], sd[p + "norm3.bias"], cfg.eps)
            x = x + self._lin(F.gelu(self._lin(n, p + "ff.net.0.proj"), approximate="tanh"), p + "ff.net.2")
        return x

    @torch.no_grad()
    def velocity(self, x: torch.Tensor, state_feat: torch.Tensor, vl: torch.Tensor, image_mask, valid_mask, s: int) -> torch.Tensor:
        cfg, sd, H = self.cfg, self.sd, self.cfg.hidden
        get = sd.__getitem__
        b = cfg.bucket(s)
        cond = timestep_cond(get, cfg, b).to(self.device)
        tau = action_time_encoding(cfg, b).to(self.device)[None].expand(cfg.horizon, -1)
        a = self._cat(x, "action_encoder.W1")
        a = F.silu(self._cat(torch.cat((a, tau), -1), "action_encoder.W2"))
        a = self._cat(a, "action_encoder.W3") + sd[AP + "position_embedding.weight"][:cfg.horizon]
        h = torch.cat((state_feat, a), 0)
        im, ok = image_mask.reshape(-1).bool().to(self.device), valid_mask.reshape(-1).bool().to(self.device)
        for i in range(cfg.layers):
            p = f"{AP}model.transformer_blocks.{i}."
            mod = self._lin(cond, p + "norm1.linear")
            n = F.layer_norm(h, (H,), eps=cfg.eps) * (1 + mod[:H]) + mod[H:]
            if i % 2 == 0:
                src = vl[((~im) & ok) if i % 4 == 0 else (im & ok)]
            else:
                src = n
            att = self._attn(self._lin(n, p + "attn1.to_q"), self._lin(src, p + "attn1.to_k"), self._lin(src, p + "attn1.to_v"),
                             cfg.heads, cfg.head_dim)
            h = h + self._lin(att, p + "attn1.to_out.0")
            n = F.layer_norm(h, (H,), eps=cfg.eps)
            h = h + self._lin(F.gelu(self._lin(n, p + "ff.net.0.proj"), approximate="tanh"), p + "ff.net.2")
        so = self._lin(cond, AP + "model.proj_out_1")
        n = F.layer_norm(h, (H,), eps=cfg.eps_out) * (1 + so[H:]) + so[:H]
        out = self._lin(n, AP + "model.proj_out_2")
        pred = self._cat(F.relu(self._cat(out, "action_decoder.layer1")), "action_decoder.layer2")
        return pred[1:]

    @torch.no_grad()
    def denoise(self, vl: torch.Tensor, state: torch.Tensor, noise: torch.Tensor, image_mask, valid_mask) -> torch.Tensor:
        """``vl [S, vl_dim]``, ``state [state_dim]``, ``noise [horizon, action_dim]`` -> actions ``[horizon, action_dim]``."""
        cfg = self.cfg
        vl = vl.float().to(self.device)
        sf = self._cat(F.relu(self._cat(state.float().to(self.device).reshape(1, -1), "state_encoder.layer1")), "state_encoder.layer2")
        x = noise.float().to(self.device).clone()
        for s in range(cfg.steps):
            x = x + (1.0 / cfg.steps) * self.velocity(x, sf, vl, image_mask, valid_mask, s)
        return x


# ----------------------------------------------------------------------------- device engine
def _r8(n: int) -> int:
    return (n + 7) // 8 * 8


class Gr00tEngine:
    """VL encoder and DiT denoise loop on the accelerator for one embodiment and VL sequences of up to ``max_vl`` tokens."""

    def __init__(self, cfg: Gr00tConfig, get, *, embodiment: int = 0, max_vl: int = 512, device="cuda", dtype=torch.float16):
        from ..ops import kernels as K
        from ..runtime.stack import pad_heads
        self.K, self.cfg, self.device, self.dtype, self.max_vl, self.emb = K, cfg, torch.device(device), dtype, max_vl, embodiment
        check_state_dict(cfg, get)
        if not 0 <= embodiment < cfg.embodiments:
            raise ValueError(f"embodiment {embodiment} is outside the checkpoint's {cfg.embodiments} banks")
        dev, H = self.device, cfg.hidden
        t = lambda w: w.to(dev, dtype).contiguous()
        pack = lambda w: K.pack_weight(t(w))
        pad = lambda hd: 64 if hd <= 64 else (128 if hd <= 128 else 256)
        self.hp, self.vhp = pad(cfg.head_dim), pad(cfg.vl_head_dim)
        self.D, self.VD = cfg.heads * self.hp, cfg.vl_heads * self.vhp
        z = lambda *s: torch.zeros(*s, dtype=dtype, device=dev)

        def attn_weights(p, heads, hd, hp, fused_qkv):
            w = {n: pad_heads(get(p + f"attn1.to_{n}.weight"), heads, hd, hp, 0) for n in "qkv"}
            b = {n: pad_heads(get(p + f"attn1.to_{n}.bias"), heads, hd, hp, 0) for n in "qkv"}
            L = {}
            if fused_qkv:
                L["qkv_w"], L["qkv_b"] = pack(torch.cat([w[n] for n in "qkv"], 0)), t(torch.cat([b[n] for n in "qkv"], 0))
            else:
                L["q_w"], L["q_b"] = pack(w["q"]), t(b["q"])
                L["kv_w"], L["kv_b"] = pack(torch.cat((w["k"], w["v"]), 0)), t(torch.cat((b["k"], b["v"]), 0))
            L["o_w"] = pack(pad_heads(get(p + "attn1.to_out.0.weight"), heads, hd, hp, 1))
            L["o_b"] = t(get(p + "attn1.to_out.0.bias"))
            L["f1_w"], L["f1_b"] = pack(get(p + "ff.net.0.proj.weight")), t(get(p + "ff.net.0.proj.bias"))
            L["f2_w"], L["f2_b"] = pack(get(p + "ff.net.2.weight")), t(get(p + "ff.net.2.bias"))
            return L

        # ---- VL encoder
        self.vlln_w, self.vlln_b = t(get(AP + "vlln.weight")), t(get(AP + "vlln.bias"))
        self.vl_layers = []
        for i in range(cfg.vl_layers):
            p = f"{AP}vl_self_attention.transformer_blocks.{i}."
            L = attn_weights(p, cfg.vl_heads, cfg.vl_head_dim, self.vhp, True)
            for n in ("norm1", "norm3"):
                L[n + "_w"], L[n + "_b"] = t(get(p + n + ".weight")), t(get(p + n + ".bias"))
            self.vl_layers.append(L)
        S = max_vl
        self.vx, self.vn, self.vqkv, self.vatt, self.vff = z(S, cfg.vl_dim), z(S, cfg.vl_dim), z(S, 3 * self.VD), z(S, self.VD), z(S, cfg.vl_ff)
        self.vl_sorted = z(S, cfg.vl_dim)

        # ---- DiT blocks and the modulation tables of every (step, block)
        cond = torch.stack([timestep_cond(get, cfg, cfg.bucket(s)) for s in range(cfg.steps)])          # [steps, H] fp32
        self.layers = []
        mod_w, mod_b = [], []
        for i in range(cfg.layers):
            p = f"{AP}model.transformer_blocks.{i}."
            self.layers.append(attn_weights(p, cfg.heads, cfg.head_dim, self.hp, i % 2 == 1))
            m = F.linear(cond, get(p + "norm1.linear.weight").float(), get(p + "norm1.linear.bias").float())   # [steps, 2H]
            mod_w.append(1.0 + m[:, :H])
            mod_b.append(m[:, H:])
        self.mod_w, self.mod_b = t(torch.stack(mod_w, 1)), t(torch.stack(mod_b, 1))                   # [steps, layers, H]
        so = F.linear(cond, get(AP + "model.proj_out_1.weight").float(), get(AP + "model.proj_out_1.bias").float())
        self.out_w, self.out_b = t(1.0 + so[:, H:]), t(so[:, :H])
        self.ones, self.zeros = torch.ones(H, dtype=dtype, device=dev), z(H)

        # ---- per-embodiment encoders / decoder ([in, out] banks -> [out, in] rows; odd widths padded to 8)
        e = embodiment
        bank = lambda n: get(AP + n + ".W")[e].float().t().contiguous()
        bias = lambda n: get(AP + n + ".b")[e].float()
        self.a_pad, self.s_pad = _r8(cfg.action_dim), _r8(cfg.state_dim)
        self.se1_w, self.se1_b = t(F.pad(bank("state_encoder.layer1"), (0, self.s_pad - cfg.state_dim))), t(bias("state_encoder.layer1"))
        self.se2_w, self.se2_b = pack(bank("state_encoder.layer2")), t(bias("state_encoder.layer2"))
        self.ae1_w, self.ae1_b = t(F.pad(bank("action_encoder.W1"), (0, self.a_pad - cfg.action_dim))), t(bias("action_encoder.W1"))
        self.ae2_w, self.ae2_b = pack(bank("action_encoder.W2")), t(bias("action_encoder.W2"))
        self.ae3_w, self.ae3_b = pack(bank("action_encoder.W3")), t(bias("action_encoder.W3"))
        self.po2_w, self.po2_b = pack(get(AP + "model.proj_out_2.weight")), t(get(AP + "model.proj_out_2.bias"))
        self.d1_w, self.d1_b = pack(bank("action_decoder.layer1")), t(bias("action_decoder.layer1"))
        self.d2_w = t(F.pad(bank("action_decoder.layer2"), (0, 0, 0, self.a_pad - cfg.action_dim)))
        self.d2_b = t(F.pad(bias("action_decoder.layer2"), (0, self.a_pad - cfg.action_dim)))
        A, Q = cfg.horizon, cfg.horizon + 1
        self.pos = t(get(AP + "position_embedding.weight")[:A])
        # the action encoder's second layer reads [a_emb | sincos(t_s)]: one buffer per step with the right half filled
        self.enc_in = z(cfg.steps, A, 2 * H)
        for s in range(cfg.steps):
            self.enc_in[s, :, H:] = action_time_encoding(cfg, cfg.bucket(s)).to(dev, dtype)[None]
        self.x, self.state = z(A, self.a_pad), z(1, self.s_pad)
        self.se_mid, self.state_feat, self.enc_mid = z(1, cfg.enc_mid), z(1, H), z(A, H)
        self.h, self.hn, self.q, self.qkv, self.att, self.ffb = z(Q, H), z(Q, H), z(Q, self.D), z(Q, 3 * self.D), z(Q, self.D), z(Q, cfg.ff)
        self.mo, self.dm, self.pred = z(Q, cfg.model_out), z(Q, cfg.dec_mid), z(Q, self.a_pad)
        self.cross_kv = {i: z(S, 2 * self.D) for i in range(0, cfg.layers, 2)}
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        self.q_start, self.q_len = i32([0]), i32([Q])
        self.kv_self = i32([Q])
        self.kv_text_start, self.kv_text_len, self.kv_img_start, self.kv_img_len = i32([0]), i32([0]), i32([0]), i32([0])
        self.vl_q_len = i32([0])
        self.status = torch.zeros(32, dtype=torch.int32, device=dev)
        self._graph: Optional[torch.cuda.CUDAGraph] = None

    # ---- VL encoder -------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def vl_encode(self, hidden: torch.Tensor, *, inv_norm_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``hidden [S, vl_dim]``: the backbone's residual stream at the selected layer -> VL embeddings ``[S, vl_dim]``
        (a view of an engine buffer).  A caller that only has the stream after the backbone's final RMSNorm passes
        ``inv_norm_weight = 1 / norm.weight``: LayerNorm does not see the per-row RMS, so dividing the weight out
        restores the same input."""
        cfg, K = self.cfg, self.K
        S = hidden.shape[0]
        if S > self.max_vl or hidden.shape[1] != cfg.vl_dim:
            raise ValueError(f"hidden must be [<= {self.max_vl}, {cfg.vl_dim}], got {tuple(hidden.shape)}")
        src = hidden.to(self.device, self.dtype)
        if inv_norm_weight is not None:
            src = src * inv_norm_weight.to(self.device, self.dtype)
        x, n, qkv, att, ff = self.vx[:S], self.vn[:S], self.vqkv[:S], self.vatt[:S], self.vff[:S]
        K.layernorm(src.contiguous(), self.vlln_w, self.vlln_b, cfg.eps, out=x)
        self.vl_q_len.fill_(S)
        VD = self.VD
        for L in self.vl_layers:
            K.layernorm(x, L["norm1_w"], L["norm1_b"], cfg.eps, out=n)
            K.gemm(n, L["qkv_w"], packed_shape=(3 * VD, cfg.vl_dim), bias=L["qkv_b"], out=qkv)
            K.attention_prefill(qkv[:, :VD], att, Hq=cfg.vl_heads, Hkv=cfg.vl_heads, hd=self.vhp, q_start=self.q_start, q_len=self.vl_q_len,
                                kv_len=self.vl_q_len, max_q_len=S, k=qkv[:, VD:2 * VD], v=qkv[:, 2 * VD:], kv_start=self.q_start,
                                causal=False, scale=1.0 / math.sqrt(cfg.vl_head_dim), status=self.status, max_kv_len=S)
            K.gemm(att, L["o_w"], packed_shape=(cfg.vl_dim, VD), bias=L["o_b"], residual=x, out=x)
            K.layernorm(x, L["norm3_w"], L["norm3_b"], cfg.eps, out=n)
            K.gemm(n, L["f1_w"], packed_shape=(cfg.vl_ff, cfg.vl_dim), bias=L["f1_b"], act="gelu_tanh", out=ff)
            K.gemm(ff, L["f2_w"], packed_shape=(cfg.vl_dim, cfg.vl_ff), bias=L["f2_b"], residual=x, out=x)
        return x

    # ---- DiT --------------------------------------------------------------------------------------------------------
    def _tail(self, L) -> None:
        cfg, K, H = self.cfg, self.K, self.cfg.hidden
        K.gemm(self.att, L["o_w"], packed_shape=(H, self.D), bias=L["o_b"], residual=self.h, out=self.h)
        K.layernorm(self.h, self.ones, self.zeros, cfg.eps, out=self.hn)
        K.gemm(self.hn, L["f1_w"], packed_shape=(cfg.ff, H), bias=L["f1_b"], act="gelu_tanh", out=self.ffb)
        K.gemm(self.ffb, L["f2_w"], packed_shape=(H, cfg.ff), bias=L["f2_b"], residual=self.h, out=self.h)

    def _step(self, s: int) -> None:
        cfg, K, H, D = self.cfg, self.K, self.cfg.hidden, self.D
        A, Q = cfg.horizon, cfg.horizon + 1
        scale = 1.0 / math.sqrt(cfg.head_dim)
        K.gemm(self.x, self.ae1_w, bias=self.ae1_b, out=self.enc_in[s, :, :H])
        K.gemm(self.enc_in[s], self.ae2_w, packed_shape=(H, 2 * H), bias=self.ae2_b, act="silu", out=self.enc_mid)
        K.gemm(self.enc_mid, self.ae3_w, packed_shape=(H, H), bias=self.ae3_b, residual=self.pos, out=self.h[1:])
        self.h[0:1].copy_(self.state_feat)
        for i, L in enumerate(self.layers):
            K.layernorm(self.h, self.mod_w[s, i], self.mod_b[s, i], cfg.eps, out=self.hn)
            if i % 2 == 0:
                kv = self.cross_kv[i]
                K.gemm(self.hn, L["q_w"], packed_shape=(D, H), bias=L["q_b"], out=self.q)
                text = i % 4 == 0
                K.attention_prefill(self.q, self.att, Hq=cfg.heads, Hkv=cfg.heads, hd=self.hp, q_start=self.q_start, q_len=self.q_len,
                                    kv_len=self.kv_text_len if text else self.kv_img_len, max_q_len=Q, k=kv[:, :D], v=kv[:, D:],
                                    kv_start=self.kv_text_start if text else self.kv_img_start, causal=False, scale=scale,
                                    status=self.status, max_kv_len=self.max_vl)
            else:
                K.gemm(self.hn, L["qkv_w"], packed_shape=(3 * D, H), bias=L["qkv_b"], out=self.qkv)
                K.attention_prefill(self.qkv[:, :D], self.att, Hq=cfg.heads, Hkv=cfg.heads, hd=self.hp, q_start=self.q_start,
                                    q_len=self.q_len, kv_len=self.kv_self, max_q_len=Q, k=self.qkv[:, D:2 * D], v=self.qkv[:, 2 * D:],
                                    kv_start=self.q_start, causal=False, scale=scale, status=self.status, max_kv_len=Q)
            self._tail(L)
        K.layernorm(self.h, self.out_w[s], self.out_b[s], cfg.eps_out, out=self.hn)
        K.gemm(self.hn, self.po2_w, packed_shape=(cfg.model_out, H), bias=self.po2_b, out=self.mo)
        K.gemm(self.mo, self.d1_w, packed_shape=(cfg.dec_mid, cfg.model_out), bias=self.d1_b, out=self.dm)
        self.dm.clamp_min_(0.0)
        K.gemm(self.dm, self.d2_w, bias=self.d2_b, out=self.pred)
        self.x.add_(self.pred[1:], alpha=1.0 / cfg.steps)

    def _loop(self) -> None:
        """State encoder, the sixteen K/V projections of the sorted VL rows (all ``max_vl`` rows: rows past the call's
        length are never attended), then the Euler steps."""
        cfg, K, H, D = self.cfg, self.K, self.cfg.hidden, self.D
        K.gemm(self.state, self.se1_w, bias=self.se1_b, out=self.se_mid)
        self.se_mid.clamp_min_(0.0)
        K.gemm(self.se_mid, self.se2_w, packed_shape=(H, cfg.enc_mid), bias=self.se2_b, out=self.state_feat)
        for i in range(0, cfg.layers, 2):
            L = self.layers[i]
            K.gemm(self.vl_sorted, L["kv_w"], packed_shape=(2 * D, cfg.vl_dim), bias=L["kv_b"], out=self.cross_kv[i])
        for s in range(cfg.steps):
            self._step(s)

    @torch.no_grad()
    def denoise(self, vl: torch.Tensor, state: torch.Tensor, noise: torch.Tensor, image_mask: torch.Tensor,
                valid_mask: Optional[torch.Tensor] = None, *, use_graph: bool = True) -> torch.Tensor:
        """``vl [S, vl_dim]`` (device), ``state [state_dim]``, ``noise [horizon, action_dim]``, ``image_mask [S]`` (True at image
        tokens), ``valid_mask [S]`` (default all) -> actions ``[horizon, action_dim]`` fp32 (a fresh device tensor)."""
        cfg, dev = self.cfg, self.device
        S = vl.shape[0]
        if S > self.max_vl:
            raise ValueError(f"{S} VL tokens exceed the engine's {self.max_vl}")
        if valid_mask is None:
            valid_mask = torch.ones(S, dtype=torch.bool)
        order, n_text, n_img = subset_order(image_mask, valid_mask)
        if n_text == 0 or n_img == 0:
            raise ValueError("the cross-attention blocks need at least one text token and one image token")
        n = order.numel()
        torch.index_select(vl.to(dev, self.dtype), 0, order.to(dev), out=self.vl_sorted[:n])
        meta = torch.tensor([0, n_text, n_text, n_img], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        self.kv_text_start.copy_(meta[0:1]); self.kv_text_len.copy_(meta[1:2])
        self.kv_img_start.copy_(meta[2:3]); self.kv_img_len.copy_(meta[3:4])
        self.state.zero_()
        self.state[0, :cfg.state_dim].copy_(state.reshape(-1).to(dev, self.dtype))
        self.x.zero_()
        self.x[:, :cfg.action_dim].copy_(noise.reshape(cfg.horizon, cfg.action_dim).to(dev, self.dtype))
        if not use_graph:
            self._loop()
        else:
            if self._graph is None:
                snap = self.x.clone()
                st = torch.cuda.Stream()
                st.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(st):
                    self._loop()
                torch.cuda.current_stream().wait_stream(st)
                self.x.copy_(snap)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    self._loop()
                torch.cuda.synchronize()
                self.x.copy_(snap)
                self._graph = g
            self._graph.replay()
        return self.x[:, :cfg.action_dim].float().clone()

    def check_status(self) -> None:
        torch.cuda.synchronize()
        st = self.status.tolist()
        if st[0] != 0:
            from ..runtime.errors import RPUBackendError
            raise RPUBackendError(f"device status {st[:4]} (code, block, kernel, detail)")

    def close(self) -> None:
        self._graph = None


__all__ = ["Gr00tConfig", "Gr00tEngine", "TorchGr00t", "tiny_gr00t_config", "gr00t_shapes", "random_gr00t_state_dict",
           "check_state_dict", "timestep_cond", "action_time_encoding", "subset_order", "AP"]
