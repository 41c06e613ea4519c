"""InternVLA-N1 trajectory head: a 12-block Lumina NextDiT over 32 action tokens, conditioned on the language system's
latent tokens, integrated with a fixed flow-matching Euler schedule.

One block, with ``temb = time_embed(t) + caption_embed(mean(caption))`` and
``[scale_msa, gate_msa, scale_mlp, gate_mlp] = Linear(silu(temb))``::

    n     = RMSNorm(x; norm1) (1 + scale_msa)
    self  = SDPA(LN_H(n Wq), LN_H(n Wk), n Wv)                        # LayerNorm over all 384 channels, then 6 heads of 64
    cross = SDPA(LN_H(n Wq'), LN_H(ctx Wk'), ctx Wv') * tanh(gate_h)   # ctx = RMSNorm(caption; norm1_context)
    x     = x + tanh(gate_msa) RMSNorm((self + cross) Wo; norm2)
    f     = RMSNorm(x; ffn_norm1) (1 + scale_mlp)
    x     = x + tanh(gate_mlp) RMSNorm(W2 (silu(W1 f) * W3 f); ffn_norm2)

and the head ``raw = D (L2 (LN(x) (1 + Linear(silu(temb)))))``, ``actions += euler_step * raw``.

What is hoisted here:

* per condition: the caption projection, one weight-free RMSNorm shared by all blocks (every block's context-norm weight
  is folded into the columns of its K / V projection), and all twelve cross K / V projections with the per-head
  ``tanh(gate)`` folded into the V rows; the cross keys get their full-width LayerNorm once;
* per call: the modulation of every (step, block) as one small GEMM, multiplied into the four RMSNorm weights of each
  block, so a modulated or gated norm is one plain RMSNorm launch with a per-step weight row;
* per block: self Q / K / V and cross Q come out of ONE GEMM; self and cross outputs sit side by side so the shared
  output projection (its weight duplicated along K) adds them.

The Euler loop over up to four trajectories (packed as rows; self-attention per trajectory, one shared cross cache)
replays from one CUDA graph per (batch, step count); schedules, conditions and caption lengths change without a new capture.

Reference behaviour: ``src/fused/rpu_internvla_nextdit_model.cpp:1-17,760-1015`` (block and head),
``python/rpu_backend/adapters/internvla_n1/nextdit.py:128-306`` (condition and step glue), ``:554-625`` (tensor names),
``:1150-1250`` (Euler schedule call).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterator, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass
class NextDiTConfig:
    layers: int = 12
    hidden: int = 384
    heads: int = 6
    head_dim: int = 64
    ff: int = 1536
    cond_dim: int = 384             # width of the incoming condition tokens
    freq_dim: int = 256             # sinusoidal width of the timestep embedder
    action_seq: int = 32
    action_dim: int = 3
    eps: float = 1e-5
    final_eps: float = 1e-6
    qk_eps: float = 1e-5
    max_cross: int = 320
    max_batch: int = 4
    max_steps: int = 10

    @property
    def temb_dim(self) -> int:
        return min(self.hidden, 1024)


def tiny_nextdit_config(**kw) -> NextDiTConfig:
    base = dict(layers=2, hidden=128, heads=2, head_dim=64, ff=256, cond_dim=96, freq_dim=32, action_seq=8, max_cross=24)
    base.update(kw)
    return NextDiTConfig(**base)


def nextdit_shapes(cfg: NextDiTConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    H, T = cfg.hidden, cfg.temb_dim
    yield "model.caption_projection.weight", (H, cfg.cond_dim), "matrix"
    yield "model.caption_projection.bias", (H,), "bias"
    te = "model.time_caption_embed."
    yield te + "timestep_embedder.linear_1.weight", (T, cfg.freq_dim), "matrix"
    yield te + "timestep_embedder.linear_1.bias", (T,), "bias"
    yield te + "timestep_embedder.linear_2.weight", (T, T), "matrix"
    yield te + "timestep_embedder.linear_2.bias", (T,), "bias"
    yield te + "caption_embedder.0.weight", (H,), "norm"
    yield te + "caption_embedder.0.bias", (H,), "bias"
    yield te + "caption_embedder.1.weight", (T, H), "matrix"
    yield te + "caption_embedder.1.bias", (T,), "bias"
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        for a in ("attn1", "attn2"):
            for n in ("to_q", "to_k", "to_v"):
                yield p + f"{a}.{n}.weight", (H, H), "matrix"
            for n in ("norm_q", "norm_k"):
                yield p + f"{a}.{n}.weight", (H,), "norm"
                yield p + f"{a}.{n}.bias", (H,), "bias"
        yield p + "attn2.to_out.0.weight", (H, H), "matrix"
        yield p + "gate", (cfg.heads,), "gate"
        yield p + "feed_forward.linear_1.weight", (cfg.ff, H), "matrix"
        yield p + "feed_forward.linear_2.weight", (H, cfg.ff), "matrix"
        yield p + "feed_forward.linear_3.weight", (cfg.ff, H), "matrix"
        yield p + "norm1.linear.weight", (4 * H, T), "small"
        yield p + "norm1.linear.bias", (4 * H,), "bias"
        for n in ("norm1.norm", "norm2", "ffn_norm1", "ffn_norm2", "norm1_context"):
            yield p + n + ".weight", (H,), "norm"
    yield "model.norm_out.linear_1.weight", (H, T), "small"
    yield "model.norm_out.linear_1.bias", (H,), "bias"
    yield "model.norm_out.linear_2.weight", (H, H), "matrix"
    yield "model.norm_out.linear_2.bias", (H,), "bias"
    yield "action_encoder.weight", (H, cfg.action_dim), "matrix"
    yield "action_encoder.bias", (H,), "bias"
    yield "action_position", (cfg.action_seq, H), "embed"
    yield "action_decoder.weight", (cfg.action_dim, H), "matrix"
    yield "action_decoder.bias", (cfg.action_dim,), "bias"


def random_nextdit_state_dict(cfg: NextDiTConfig, *, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in nextdit_shapes(cfg):
        r = torch.randn(shape, generator=g)
        sd[name] = {"matrix": r / math.sqrt(shape[-1]), "small": r * 0.3 / math.sqrt(shape[-1]), "embed": r * 0.2,
                    "norm": 1.0 + 0.05 * r, "bias": 0.03 * r, "gate": 0.5 * r}[kind]
    return sd


def check_state_dict(cfg: NextDiTConfig, sd) -> None:
    bad = []
    for name, shape, _ in nextdit_shapes(cfg):
        if name not in sd:
            bad.append(f"{name}: missing")
        elif tuple(sd[name].shape) != shape:
            bad.append(f"{name}: {tuple(sd[name].shape)}, expected {shape}")
    if bad:
        raise ValueError(f"NextDiT weights do not fit the {cfg.layers}-block profile ({len(bad)} tensors): " + "; ".join(bad[:6]))


def time_frequencies(t: torch.Tensor, dim: int) -> torch.Tensor:
    """Cos-first sinusoid of ``t`` (no frequency shift): ``[len(t), dim]`` fp32."""
    half = dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    a = t.float().reshape(-1, 1) * f[None]
    return torch.cat((a.cos(), a.sin()), -1)


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


# ----------------------------------------------------------------------------- fp32 oracle
class TorchNextDiT:
    def __init__(self, cfg: NextDiTConfig, sd: Dict[str, torch.Tensor], device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.sd = {k: v.float().to(self.device) for k, v in sd.items()}

    def _sdpa(self, q, k, v):
        c = self.cfg
        sp = lambda t: t.reshape(t.shape[0], c.heads, c.head_dim).transpose(0, 1)
        return F.scaled_dot_product_attention(sp(q), sp(k), sp(v)).transpose(0, 1).reshape(q.shape[0], c.hidden)

    @torch.no_grad()
    def temb(self, t: torch.Tensor, caption: torch.Tensor) -> torch.Tensor:
        sd, c = self.sd, self.cfg
        te = "model.time_caption_embed."
        f = time_frequencies(t.to(self.device), c.freq_dim)
        h = F.silu(F.linear(f, sd[te + "timestep_embedder.linear_1.weight"], sd[te + "timestep_embedder.linear_1.bias"]))
        h = F.linear(h, sd[te + "timestep_embedder.linear_2.weight"], sd[te + "timestep_embedder.linear_2.bias"])
        pool = caption.mean(0, keepdim=True)
        pool = F.layer_norm(pool, (c.hidden,), sd[te + "caption_embedder.0.weight"], sd[te + "caption_embedder.0.bias"])
        return h + F.linear(pool, sd[te + "caption_embedder.1.weight"], sd[te + "caption_embedder.1.bias"])

    @torch.no_grad()
    def velocity(self, actions: torch.Tensor, t: float, condition: torch.Tensor) -> torch.Tensor:
        """``actions [seq, action_dim]``, ``condition [S, cond_dim]`` -> raw action update ``[seq, action_dim]``."""
        sd, c, H = self.sd, self.cfg, self.cfg.hidden
        caption = F.linear(condition.float().to(self.device), sd["model.caption_projection.weight"], sd["model.caption_projection.bias"])
        temb = self.temb(torch.tensor([t]), caption)
        x = F.linear(actions.float().to(self.device), sd["action_encoder.weight"], sd["action_encoder.bias"]) + sd["action_position"]
        for i in range(c.layers):
            p = f"model.layers.{i}."
            m = F.linear(F.silu(temb), sd[p + "norm1.linear.weight"], sd[p + "norm1.linear.bias"])[0]
            scale_msa, gate_msa, scale_mlp, gate_mlp = m.chunk(4)
            n = _rms(x, sd[p + "norm1.norm.weight"], c.eps) * (1 + scale_msa)
            ln = lambda v, nm: F.layer_norm(v, (H,), sd[p + nm + ".weight"], sd[p + nm + ".bias"], c.qk_eps)
            so = self._sdpa(ln(n @ sd[p + "attn1.to_q.weight"].t(), "attn1.norm_q"), ln(n @ sd[p + "attn1.to_k.weight"].t(), "attn1.norm_k"),
                            n @ sd[p + "attn1.to_v.weight"].t())
            ctx = _rms(caption, sd[p + "norm1_context.weight"], c.eps)
            co = self._sdpa(ln(n @ sd[p + "attn2.to_q.weight"].t(), "attn2.norm_q"), ln(ctx @ sd[p + "attn2.to_k.weight"].t(), "attn2.norm_k"),
                            ctx @ sd[p + "attn2.to_v.weight"].t())
            co = (co.reshape(-1, c.heads, c.head_dim) * sd[p + "gate"].tanh()[None, :, None]).reshape(-1, H)
            a = (so + co) @ sd[p + "attn2.to_out.0.weight"].t()
            x = x + gate_msa.tanh() * _rms(a, sd[p + "norm2.weight"], c.eps)
            f = _rms(x, sd[p + "ffn_norm1.weight"], c.eps) * (1 + scale_mlp)
            ff = (F.silu(f @ sd[p + "feed_forward.linear_1.weight"].t()) * (f @ sd[p + "feed_forward.linear_3.weight"].t())) \
                @ sd[p + "feed_forward.linear_2.weight"].t()
            x = x + gate_mlp.tanh() * _rms(ff, sd[p + "ffn_norm2.weight"], c.eps)
        fs = 1 + F.linear(F.silu(temb), sd["model.norm_out.linear_1.weight"], sd["model.norm_out.linear_1.bias"])[0]
        x = F.layer_norm(x, (H,), eps=c.final_eps) * fs
        x = F.linear(x, sd["model.norm_out.linear_2.weight"], sd["model.norm_out.linear_2.bias"])
        return F.linear(x, sd["action_decoder.weight"], sd["action_decoder.bias"])

    @torch.no_grad()
    def denoise_actions(self, actions: torch.Tensor, timesteps: Sequence[float], euler_steps: Sequence[float], condition: torch.Tensor):
        x = actions.float().to(self.device).clone()
        for t, dt in zip(timesteps, euler_steps):
            x = torch.stack([x[b] + float(dt) * self.velocity(x[b], float(t), condition) for b in range(x.shape[0])])
        return x


# ----------------------------------------------------------------------------- device engine
class NextDiTEngine:
    def __init__(self, cfg: NextDiTConfig, sd: Dict[str, torch.Tensor], *, device="cuda", dtype=torch.float16):
        from ..ops import kernels as K
        check_state_dict(cfg, sd)
        if cfg.head_dim not in (64, 128, 256) or cfg.heads * cfg.head_dim != cfg.hidden:
            raise ValueError(f"NextDiT geometry {cfg.heads} x {cfg.head_dim} over {cfg.hidden} is outside the attention kernels")
        self.K, self.cfg, self.device, self.dtype = K, cfg, torch.device(device), dtype
        dev, H, T, NL = self.device, cfg.hidden, cfg.temb_dim, cfg.layers
        t = lambda w: w.to(dev, dtype).contiguous()
        f32 = lambda w: w.float().to(dev).contiguous()
        pack = lambda w: K.pack_weight(t(w))
        z = lambda *s: torch.zeros(*s, dtype=dtype, device=dev)
        self.layers = []
        for i in range(NL):
            p = f"model.layers.{i}."
            g = lambda n: sd[p + n].float()
            L = {}
            L["qkqv_w"] = pack(torch.cat((g("attn1.to_q.weight"), g("attn1.to_k.weight"), g("attn2.to_q.weight"), g("attn1.to_v.weight")), 0))
            cw = g("norm1_context.weight")[None, :]
            gate = g("gate").tanh().repeat_interleave(cfg.head_dim)[:, None]
            L["ckv_w"] = pack(torch.cat((g("attn2.to_k.weight") * cw, g("attn2.to_v.weight") * cw * gate), 0))
            L["o_w"] = pack(torch.cat((g("attn2.to_out.0.weight"),) * 2, 1))
            L["ff13_w"] = K.pack_weight(t(torch.cat((g("feed_forward.linear_1.weight"), g("feed_forward.linear_3.weight")), 0)), sections=2)
            L["ff2_w"] = pack(g("feed_forward.linear_2.weight"))
            for key, n in (("sq", "attn1.norm_q"), ("sk", "attn1.norm_k"), ("cq", "attn2.norm_q"), ("ck", "attn2.norm_k")):
                L[key + "_w"], L[key + "_b"] = t(g(n + ".weight")), t(g(n + ".bias"))
            self.layers.append(L)
        # fp32 glue that runs once per call on the device
        te = "model.time_caption_embed."
        self.glue = {k: f32(sd[k]) for k in (te + "timestep_embedder.linear_1.weight", te + "timestep_embedder.linear_1.bias",
                                             te + "timestep_embedder.linear_2.weight", te + "timestep_embedder.linear_2.bias",
                                             te + "caption_embedder.0.weight", te + "caption_embedder.0.bias",
                                             te + "caption_embedder.1.weight", te + "caption_embedder.1.bias")}
        self.mod_w = f32(torch.cat([sd[f"model.layers.{i}.norm1.linear.weight"] for i in range(NL)] + [sd["model.norm_out.linear_1.weight"]], 0))
        self.mod_b = f32(torch.cat([sd[f"model.layers.{i}.norm1.linear.bias"] for i in range(NL)] + [sd["model.norm_out.linear_1.bias"]], 0))
        # [layers, 4, H]: the learned weights of norm1 / norm2 / ffn_norm1 / ffn_norm2 in modulation order
        self.norm_w = f32(torch.stack([torch.stack([sd[f"model.layers.{i}.{n}.weight"] for n in ("norm1.norm", "norm2", "ffn_norm1", "ffn_norm2")])
                                       for i in range(NL)]))
        self.cap_w, self.cap_b = pack(sd["model.caption_projection.weight"]), t(sd["model.caption_projection.bias"])
        self.c_pad = (cfg.cond_dim + 7) // 8 * 8
        if self.c_pad != cfg.cond_dim:
            self.cap_w = pack(F.pad(sd["model.caption_projection.weight"].float(), (0, self.c_pad - cfg.cond_dim)))
        self.a_pad = (cfg.action_dim + 7) // 8 * 8
        self.enc_w, self.enc_b = t(F.pad(sd["action_encoder.weight"].float(), (0, self.a_pad - cfg.action_dim))), t(sd["action_encoder.bias"])
        self.dec_w = t(F.pad(sd["action_decoder.weight"].float(), (0, 0, 0, self.a_pad - cfg.action_dim)))
        self.dec_b = t(F.pad(sd["action_decoder.bias"].float(), (0, self.a_pad - cfg.action_dim)))
        self.out_w, self.out_b = pack(sd["model.norm_out.linear_2.weight"]), t(sd["model.norm_out.linear_2.bias"])
        B, P, S, NS = cfg.max_batch, cfg.action_seq, cfg.max_cross, cfg.max_steps
        R = B * P
        self.pos = t(sd["action_position"]).repeat(B, 1)
        self.ones, self.zeros = torch.ones(H, dtype=dtype, device=dev), z(H)
        self.cond_in, self.caption, self.ctx = z(S, self.c_pad), z(S, H), z(S, H)
        self.cross_kv = [z(S, 2 * H) for _ in range(NL)]
        self.tab = z(NS, NL, 4, H)                       # per-step RMSNorm weight rows
        self.final_scale = z(NS, H)
        self.dt = torch.zeros(NS, dtype=dtype, device=dev)
        self.x, self.raw = z(R, self.a_pad), z(R, self.a_pad)
        self.h, self.n, self.qkqv, self.att, self.a, self.tmp = z(R, H), z(R, H), z(R, 4 * H), z(R, 2 * H), z(R, H), z(R, H)
        self.ffb = z(R, cfg.ff)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        self.meta = {b: dict(q_start=i32([j * P for j in range(b)]), q_len=i32([P] * b), zero=i32([0] * b)) for b in range(1, B + 1)}
        self.cross_len = i32([0] * B)
        self.status = torch.zeros(32, dtype=torch.int32, device=dev)
        self._graphs: Dict[Tuple[int, int], torch.cuda.CUDAGraph] = {}
        self._cond_key = None
        self._caption_embedding: Optional[torch.Tensor] = None

    # ---- per condition ----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def set_condition(self, condition: torch.Tensor, *, reuse: bool = True) -> None:
        """``condition [S, cond_dim]`` (or ``[1, S, cond_dim]``): caption projection, pooled caption embedding and the cross
        K / V of every block.  With ``reuse`` an identical tensor is recognised and skipped."""
        cfg, K, H = self.cfg, self.K, self.cfg.hidden
        cond = condition.reshape(-1, condition.shape[-1])
        S = cond.shape[0]
        if S > cfg.max_cross or S < 1 or cond.shape[1] != cfg.cond_dim:
            raise ValueError(f"condition must be [1..{cfg.max_cross}, {cfg.cond_dim}], got {tuple(cond.shape)}")
        if reuse and self._cond_key is not None and self._cond_key.shape == cond.shape and torch.equal(self._cond_key, cond):
            return
        self._cond_key = cond.detach().clone() if reuse else None
        self.cond_in[:S, :cfg.cond_dim].copy_(cond.to(self.device, self.dtype))
        K.gemm(self.cond_in[:S], self.cap_w, packed_shape=(H, self.c_pad), bias=self.cap_b, out=self.caption[:S])
        g, te = self.glue, "model.time_caption_embed."
        pool = self.caption[:S].float().mean(0, keepdim=True)
        pool = F.layer_norm(pool, (H,), g[te + "caption_embedder.0.weight"], g[te + "caption_embedder.0.bias"])
        self._caption_embedding = F.linear(pool, g[te + "caption_embedder.1.weight"], g[te + "caption_embedder.1.bias"])
        K.rmsnorm(self.caption[:S], None, cfg.eps, out=self.ctx[:S])
        for L, kv in zip(self.layers, self.cross_kv):
            K.gemm(self.ctx[:S], L["ckv_w"], packed_shape=(2 * H, H), out=kv[:S])
            K.layernorm(kv[:S, :H], L["ck_w"], L["ck_b"], cfg.qk_eps, out=kv[:S, :H])
        self.cross_len.fill_(S)

    # ---- per call ---------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def set_schedule(self, timesteps: torch.Tensor, euler_steps: torch.Tensor) -> int:
        """Modulation tables of every (step, block) for the current condition; returns the step count."""
        cfg, g, H, NL = self.cfg, self.glue, self.cfg.hidden, self.cfg.layers
        if self._caption_embedding is None:
            raise RuntimeError("set_condition() has not run")
        ts = timesteps.reshape(-1).float()
        n = ts.numel()
        if not 1 <= n <= cfg.max_steps or euler_steps.numel() != n:
            raise ValueError(f"timesteps and euler_steps must have the same length in [1, {cfg.max_steps}]")
        te = "model.time_caption_embed."
        f = time_frequencies(ts.to(self.device), cfg.freq_dim)
        h = F.silu(F.linear(f, g[te + "timestep_embedder.linear_1.weight"], g[te + "timestep_embedder.linear_1.bias"]))
        temb = F.linear(h, g[te + "timestep_embedder.linear_2.weight"], g[te + "timestep_embedder.linear_2.bias"]) + self._caption_embedding
        raw = F.linear(F.silu(temb), self.mod_w, self.mod_b)                                   # [n, (4 NL + 1) H]
        m = raw[:, :NL * 4 * H].reshape(n, NL, 4, H)
        mult = torch.stack((1 + m[:, :, 0], m[:, :, 1].tanh(), 1 + m[:, :, 2], m[:, :, 3].tanh()), 2)
        self.tab[:n].copy_((mult * self.norm_w[None]).to(self.dtype))
        self.final_scale[:n].copy_((1 + raw[:, NL * 4 * H:]).to(self.dtype))
        self.dt[:n].copy_(euler_steps.reshape(-1).to(self.device, self.dtype))
        return n

    def _step(self, b: int, s: int) -> None:
        cfg, K, H = self.cfg, self.K, self.cfg.hidden
        P, R, m = cfg.action_seq, b * cfg.action_seq, self.meta[b]
        x, h, n, qkqv, att, a, tmp, ffb = self.x[:R], self.h[:R], self.n[:R], self.qkqv[:R], self.att[:R], self.a[:R], self.tmp[:R], self.ffb[:R]
        scale = 1.0 / math.sqrt(cfg.head_dim)
        K.gemm(x, self.enc_w, bias=self.enc_b, residual=self.pos[:R], out=h)
        for i, (L, kv) in enumerate(zip(self.layers, self.cross_kv)):
            K.rmsnorm(h, self.tab[s, i, 0], cfg.eps, out=n)
            K.gemm(n, L["qkqv_w"], packed_shape=(4 * H, H), out=qkqv)
            q, k, cq, v = (qkqv[:, j * H:(j + 1) * H] for j in range(4))
            K.layernorm(q, L["sq_w"], L["sq_b"], cfg.qk_eps, out=q)
            K.layernorm(k, L["sk_w"], L["sk_b"], cfg.qk_eps, out=k)
            K.layernorm(cq, L["cq_w"], L["cq_b"], cfg.qk_eps, out=cq)
            K.attention_prefill(q, att[:, :H], Hq=cfg.heads, Hkv=cfg.heads, hd=cfg.head_dim, q_start=m["q_start"], q_len=m["q_len"],
                                kv_len=m["q_len"], max_q_len=P, k=k, v=v, kv_start=m["q_start"], causal=False, scale=scale, status=self.status,
                                max_kv_len=P)
            K.attention_prefill(cq, att[:, H:], Hq=cfg.heads, Hkv=cfg.heads, hd=cfg.head_dim, q_start=m["q_start"], q_len=m["q_len"],
                                kv_len=self.cross_len[:b], max_q_len=P, k=kv[:, :H], v=kv[:, H:], kv_start=m["zero"], causal=False,
                                scale=scale, status=self.status, max_kv_len=cfg.max_cross)
            K.gemm(att, L["o_w"], packed_shape=(H, 2 * H), out=a)
            K.rmsnorm(a, self.tab[s, i, 1], cfg.eps, out=tmp)
            h.add_(tmp)
            K.rmsnorm(h, self.tab[s, i, 2], cfg.eps, out=n)
            K.gemm(n, L["ff13_w"], packed_shape=(2 * cfg.ff, H), dual=True, act="silu_mul", out=ffb)
            K.gemm(ffb, L["ff2_w"], packed_shape=(H, cfg.ff), out=a)
            K.rmsnorm(a, self.tab[s, i, 3], cfg.eps, out=tmp)
            h.add_(tmp)
        K.layernorm(h, self.final_scale[s], self.zeros, cfg.final_eps, out=n)
        K.gemm(n, self.out_w, packed_shape=(H, H), bias=self.out_b, out=a)
        K.gemm(a, self.dec_w, bias=self.dec_b, out=self.raw[:R])
        x.addcmul_(self.raw[:R], self.dt[s:s + 1])

    @torch.no_grad()
    def denoise_actions(self, actions: torch.Tensor, timesteps: torch.Tensor, euler_steps: torch.Tensor,
                        condition: Optional[torch.Tensor] = None, *, reuse_condition: bool = True, use_graph: bool = True) -> torch.Tensor:
        """``actions [B <= max_batch, action_seq, action_dim]`` -> the integrated actions, fp32, a fresh device tensor."""
        cfg = self.cfg
        b = actions.shape[0]
        if actions.dim() != 3 or not 1 <= b <= cfg.max_batch or tuple(actions.shape[1:]) != (cfg.action_seq, cfg.action_dim):
            raise ValueError(f"actions must be [1..{cfg.max_batch}, {cfg.action_seq}, {cfg.action_dim}], got {tuple(actions.shape)}")
        if condition is not None:
            self.set_condition(condition, reuse=reuse_condition)
        n = self.set_schedule(timesteps, euler_steps)
        R = b * cfg.action_seq
        self.x.zero_()
        self.x[:R, :cfg.action_dim].copy_(actions.reshape(R, cfg.action_dim).to(self.device, self.dtype))
        if not use_graph:
            for s in range(n):
                self._step(b, s)
        else:
            g = self._graphs.get((b, n))
            if g is None:
                snap = self.x.clone()
                st = torch.cuda.Stream()
                st.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(st):
                    self._step(b, 0)
                torch.cuda.current_stream().wait_stream(st)
                self.x.copy_(snap)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    for s in range(n):
                        self._step(b, s)
                torch.cuda.synchronize()
                self.x.copy_(snap)
                self._graphs[(b, n)] = g
            g.replay()
        return self.x[:R, :cfg.action_dim].float().reshape(b, cfg.action_seq, cfg.action_dim).clone()

    def check_status(self) -> None:
        torch.cuda.synchronize()
        st = self.status.tolist()
        if st[0] != 0:
            from ..runtime.errors import RPUBackendError
            raise RPUBackendError(f"device status {st[:4]} (code, block, kernel, detail)")

    def close(self) -> None:
        self._graphs.clear()


__all__ = ["NextDiTConfig", "NextDiTEngine", "TorchNextDiT", "tiny_nextdit_config", "nextdit_shapes", "random_nextdit_state_dict",
           "check_state_dict", "time_frequencies"]
