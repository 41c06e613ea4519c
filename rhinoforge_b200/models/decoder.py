"""Causal-decoder family description, random-init weights and the plain-PyTorch oracle.

``DecoderConfig`` covers the decoder-only families the fused runtime serves with one
code path (Qwen3 / Llama / Qwen3-VL text / Gemma prefix): the reference's
``CausalDecoderModel`` recipe (``src/fused/rpu_qwen3_model.h:3040-3705``).
``TorchDecoder`` is the correctness oracle: a straightforward dense-cache
implementation of the same maths in PyTorch, cross-checked against the Hugging Face
module in the tests.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Dict, Iterator, Optional, Tuple

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class DecoderConfig:
    name: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_embeddings: bool = False
    qk_norm: bool = True
    attention_bias: bool = False
    mlp: str = "swiglu"          # swiglu | geglu_tanh
    norm: str = "rms"            # rms | rms_gemma ((1 + w) weights)
    embed_scale: float = 1.0     # Gemma multiplies embeddings by sqrt(hidden)
    max_position: int = 40960
    rotary_dim: Optional[int] = None           # partial rotary; None = head_dim
    mrope_section: Optional[Tuple[int, int, int]] = None  # M-RoPE: frequency pairs per (T, H, W) axis
    mrope_interleaved: bool = True   # True: THWTHW... (Qwen3-VL); False: contiguous T.., H.., W.. ranges (Qwen2.5-VL)
    model_type: str = "qwen3"
    # hybrid decoders (Qwen3.5): per-layer mixer kinds and the Gated-DeltaNet geometry
    layer_types: Optional[Tuple[str, ...]] = None     # "full_attention" | "linear_attention"; None: all attention
    attn_gate: bool = False                           # q_proj carries a sigmoid output gate per channel
    gdn_heads_k: int = 0
    gdn_heads_v: int = 0
    gdn_dk: int = 0
    gdn_dv: int = 0
    gdn_conv: int = 4

    @property
    def rot_dim(self) -> int:
        return self.rotary_dim or self.head_dim

    def is_linear(self, layer: int) -> bool:
        return self.layer_types is not None and self.layer_types[layer] == "linear_attention"

    def profile(self) -> Tuple[int, int, int, int]:
        """(hidden, intermediate, layers, kv_heads): the admission key of the reference
        (``python/rpu_backend/adapters/qwen3.py:119-132``)."""
        return (self.hidden_size, self.intermediate_size, self.num_layers, self.num_kv_heads)

    def param_count(self) -> int:
        H, I, L = self.hidden_size, self.intermediate_size, self.num_layers
        qkv = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim * H
        o = self.num_heads * self.head_dim * H
        per = qkv + o + 3 * H * I + 2 * H + (2 * self.head_dim if self.qk_norm else 0)
        emb = self.vocab_size * H
        return L * per + emb * (1 if self.tie_embeddings else 2) + H

    @classmethod
    def from_hf(cls, hf) -> "DecoderConfig":
        g = lambda k, d=None: getattr(hf, k, d)
        rope_theta = g("rope_theta", None)
        rp = g("rope_parameters", None) or g("rope_scaling", None) or {}
        if rope_theta is None and isinstance(rp, dict):
            rope_theta = rp.get("rope_theta", 1e6)
        mt = g("model_type", "qwen3")
        mrope = None
        mrope_il = True
        if isinstance(rp, dict) and rp.get("mrope_section"):
            mrope = tuple(rp["mrope_section"])
            mrope_il = bool(rp.get("mrope_interleaved", mt.startswith("qwen3")))
        hybrid = {}
        gemma_norm = mt.startswith("gemma")
        if mt.startswith("qwen3_5"):
            hd_ = g("head_dim", None) or hf.hidden_size // hf.num_attention_heads
            prf = float(rp.get("partial_rotary_factor", 1.0)) if isinstance(rp, dict) else 1.0
            hybrid = dict(layer_types=tuple(g("layer_types")), attn_gate=True, gdn_heads_k=g("linear_num_key_heads"),
                          gdn_heads_v=g("linear_num_value_heads"), gdn_dk=g("linear_key_head_dim"),
                          gdn_dv=g("linear_value_head_dim"), gdn_conv=g("linear_conv_kernel_dim", 4),
                          rotary_dim=int(hd_ * prf))
            gemma_norm = True           # Qwen3.5 RMSNorm stores (w - 1)
        return cls(**hybrid, **dict(
            name=g("name_or_path", mt) or mt, vocab_size=hf.vocab_size, hidden_size=hf.hidden_size,
            intermediate_size=hf.intermediate_size, num_layers=hf.num_hidden_layers,
            num_heads=hf.num_attention_heads, num_kv_heads=g("num_key_value_heads", hf.num_attention_heads),
            head_dim=g("head_dim", None) or hf.hidden_size // hf.num_attention_heads,
            rms_eps=g("rms_norm_eps", 1e-6), rope_theta=float(rope_theta or 1e6),
            tie_embeddings=bool(g("tie_word_embeddings", False)),
            qk_norm=mt in ("qwen3", "qwen3_vl_text", "qwen3_vl", "qwen3_moe") or mt.startswith("qwen3_5"),
            attention_bias=bool(g("attention_bias", False)),
            mlp="geglu_tanh" if mt.startswith("gemma") else "swiglu",
            norm="rms_gemma" if gemma_norm else "rms",
            embed_scale=math.sqrt(hf.hidden_size) if mt.startswith("gemma") else 1.0,
            max_position=g("max_position_embeddings", 40960), mrope_section=mrope, mrope_interleaved=mrope_il,
            model_type=mt))


def _q3(name, H, I, L, heads, kv, tie, vocab=151936):
    return DecoderConfig(name=name, vocab_size=vocab, hidden_size=H, intermediate_size=I, num_layers=L,
                         num_heads=heads, num_kv_heads=kv, head_dim=128, tie_embeddings=tie)


PROFILES: Dict[str, DecoderConfig] = {
    "qwen3-0.6b": _q3("qwen3-0.6b", 1024, 3072, 28, 16, 8, True),
    "qwen3-1.7b": _q3("qwen3-1.7b", 2048, 6144, 28, 16, 8, True),
    "qwen3-4b": _q3("qwen3-4b", 2560, 9728, 36, 32, 8, True),
    "qwen3-8b": _q3("qwen3-8b", 4096, 12288, 36, 32, 8, False),
    "qwen3-14b": _q3("qwen3-14b", 5120, 17408, 40, 40, 8, False),
    "qwen3-32b": _q3("qwen3-32b", 5120, 25600, 64, 64, 8, False),
    "llama-3.2-1b": DecoderConfig(name="llama-3.2-1b", vocab_size=128256, hidden_size=2048, intermediate_size=8192,
                                  num_layers=16, num_heads=32, num_kv_heads=8, head_dim=64, rms_eps=1e-5,
                                  rope_theta=5e5, tie_embeddings=True, qk_norm=False, model_type="llama"),
    "qwen3-vl-2b-text": replace(_q3("qwen3-vl-2b-text", 2048, 6144, 28, 16, 8, True), rope_theta=5e6,
                                mrope_section=(24, 20, 20), model_type="qwen3_vl_text"),
    "gemma-2b-prefix": DecoderConfig(name="gemma-2b-prefix", vocab_size=257152, hidden_size=2048,
                                     intermediate_size=16384, num_layers=18, num_heads=8, num_kv_heads=1, head_dim=256,
                                     rope_theta=1e4, tie_embeddings=True, qk_norm=False, mlp="geglu_tanh",
                                     norm="rms_gemma", embed_scale=math.sqrt(2048.0), model_type="gemma"),
}


def tiny_config(**kw) -> DecoderConfig:
    base = DecoderConfig(name="tiny", vocab_size=512, hidden_size=256, intermediate_size=512, num_layers=2,
                         num_heads=4, num_kv_heads=2, head_dim=64)
    return replace(base, **kw)


# ----------------------------------------------------------------- weights ----
def weight_shapes(cfg: DecoderConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """(HF name, shape, kind) for every tensor; kind is 'linear', 'embed' or 'norm'."""
    H, I, hd = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    yield "model.embed_tokens.weight", (cfg.vocab_size, H), "embed"
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        yield p + "input_layernorm.weight", (H,), "norm"
        yield p + "self_attn.q_proj.weight", (cfg.num_heads * hd, H), "linear"
        yield p + "self_attn.k_proj.weight", (cfg.num_kv_heads * hd, H), "linear"
        yield p + "self_attn.v_proj.weight", (cfg.num_kv_heads * hd, H), "linear"
        if cfg.attention_bias:
            yield p + "self_attn.q_proj.bias", (cfg.num_heads * hd,), "bias"
            yield p + "self_attn.k_proj.bias", (cfg.num_kv_heads * hd,), "bias"
            yield p + "self_attn.v_proj.bias", (cfg.num_kv_heads * hd,), "bias"
        yield p + "self_attn.o_proj.weight", (H, cfg.num_heads * hd), "linear"
        if cfg.qk_norm:
            yield p + "self_attn.q_norm.weight", (hd,), "norm"
            yield p + "self_attn.k_norm.weight", (hd,), "norm"
        yield p + "post_attention_layernorm.weight", (H,), "norm"
        yield p + "mlp.gate_proj.weight", (I, H), "linear"
        yield p + "mlp.up_proj.weight", (I, H), "linear"
        yield p + "mlp.down_proj.weight", (H, I), "linear"
    yield "model.norm.weight", (H,), "norm"
    if not cfg.tie_embeddings:
        yield "lm_head.weight", (cfg.vocab_size, H), "linear"


def random_state_dict(cfg: DecoderConfig, *, seed: int = 0, std: float = 0.02, dtype=torch.float16,
                      device="cpu", norm_jitter: float = 0.0) -> Dict[str, torch.Tensor]:
    """Random-init weights: normal(0, std) for linears/embeddings, ones for RMSNorm weights
    (zeros for the Gemma ``(1+w)`` flavour).  One generator per tensor, keyed by ``seed`` and the
    tensor's index, so any subset (e.g. one TP shard's layers) is reproducible on its own."""
    sd: Dict[str, torch.Tensor] = {}
    dev = torch.device(device)
    for idx, (name, shape, kind) in enumerate(weight_shapes(cfg)):
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 1_000_003 + idx)
        if kind == "norm":
            base = 0.0 if cfg.norm == "rms_gemma" else 1.0
            t = torch.full(shape, base, dtype=torch.float32, device=dev)
            if norm_jitter:
                t += norm_jitter * torch.randn(shape, generator=g, device=dev)
        elif kind == "bias":
            t = torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * std
        else:
            t = torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * std
        sd[name] = t.to(dtype)
    return sd


# ------------------------------------------------------------------ oracle ----
def rope_tables(cfg: DecoderConfig, max_pos: int, device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    rot = cfg.rot_dim
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, rot, 2, dtype=torch.float32, device=device) / rot))
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None]
    return ang.cos().contiguous(), ang.sin().contiguous()


def mrope_axis_of_freq(cfg: DecoderConfig) -> Optional[torch.Tensor]:
    """Position axis (0=T, 1=H, 2=W) used by each rotary frequency under M-RoPE: interleaved ``THWTHW...TT``
    (reference kernel semantics: ``src/ops/rpu_mrope.cpp:37-124``) or contiguous ranges ``T.. H.. W..``
    (Qwen2.5-VL; ``python/rpu_backend/runtime/rope_partial.py:129,176``)."""
    if cfg.mrope_section is None:
        return None
    axis = torch.zeros(cfg.rot_dim // 2, dtype=torch.int8)
    if cfg.mrope_interleaved:
        for dim, off in ((1, 1), (2, 2)):
            axis[off:cfg.mrope_section[dim] * 3:3] = dim
    else:
        t, h = cfg.mrope_section[0], cfg.mrope_section[1]
        axis[t:t + h] = 1
        axis[t + h:] = 2
    return axis


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


class TorchDecoder:
    """Dense-cache reference implementation in plain PyTorch (any device / dtype)."""

    def __init__(self, cfg: DecoderConfig, sd: Dict[str, torch.Tensor], *, dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.sd = {k: v.to(self.device, dtype) for k, v in sd.items()}
        if cfg.tie_embeddings and "lm_head.weight" not in self.sd:
            self.sd["lm_head.weight"] = self.sd["model.embed_tokens.weight"]
        self.k: list = [None] * cfg.num_layers
        self.v: list = [None] * cfg.num_layers

    def reset(self):
        self.k = [None] * self.cfg.num_layers
        self.v = [None] * self.cfg.num_layers

    def _norm(self, x, w):
        xf = x.float()
        n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps)
        if self.cfg.norm == "rms_gemma":
            return (n * (1.0 + w.float())).to(x.dtype)
        return w * n.to(x.dtype)

    def forward(self, ids: torch.Tensor, positions: Optional[torch.Tensor] = None,
                inputs_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        """ids [B, S] -> logits [B, S, V]; appends to the dense KV cache.
        ``positions``: [B, S] (1-D rope) or [3, B, S] (M-RoPE)."""
        cfg, sd = self.cfg, self.sd
        B, S = ids.shape[:2]
        past = 0 if self.k[0] is None else self.k[0].shape[2]
        x = inputs_embeds.to(self.device, self.dtype) if inputs_embeds is not None else \
            F.embedding(ids.to(self.device), sd["model.embed_tokens.weight"])
        if cfg.embed_scale != 1.0 and inputs_embeds is None:
            x = x * torch.tensor(cfg.embed_scale, dtype=x.dtype)
        if positions is None:
            positions = torch.arange(past, past + S, device=self.device)[None].expand(B, S)
        positions = positions.to(self.device)
        cos_t, sin_t = rope_tables(cfg, int(positions.max()) + 1, self.device)
        if positions.dim() == 3:
            axis = mrope_axis_of_freq(cfg).long().to(self.device)
            f = torch.arange(cfg.rot_dim // 2, device=self.device)
            idx = positions.permute(1, 2, 0)[..., axis]           # [B, S, rot/2]
            cos, sin = cos_t[idx, f], sin_t[idx, f]
        else:
            cos, sin = cos_t[positions], sin_t[positions]          # [B, S, rot/2]
        cos = torch.cat((cos, cos), -1)[:, None].to(self.dtype)     # [B, 1, S, rot]
        sin = torch.cat((sin, sin), -1)[:, None].to(self.dtype)
        hd, Hq, Hkv, rot = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.rot_dim
        act = F.silu if cfg.mlp == "swiglu" else (lambda t: F.gelu(t, approximate="tanh"))
        for i in range(cfg.num_layers):
            p = f"model.layers.{i}."
            h = self._norm(x, sd[p + "input_layernorm.weight"])
            q = F.linear(h, sd[p + "self_attn.q_proj.weight"], sd.get(p + "self_attn.q_proj.bias"))
            k = F.linear(h, sd[p + "self_attn.k_proj.weight"], sd.get(p + "self_attn.k_proj.bias"))
            v = F.linear(h, sd[p + "self_attn.v_proj.weight"], sd.get(p + "self_attn.v_proj.bias"))
            q = q.view(B, S, Hq, hd)
            k = k.view(B, S, Hkv, hd)
            v = v.view(B, S, Hkv, hd).transpose(1, 2)
            if cfg.qk_norm:
                q = self._norm(q, sd[p + "self_attn.q_norm.weight"])
                k = self._norm(k, sd[p + "self_attn.k_norm.weight"])
            q, k = q.transpose(1, 2), k.transpose(1, 2)

            def rope(t):
                r = t[..., :rot] * cos + _rotate_half(t[..., :rot]) * sin
                return torch.cat((r, t[..., rot:]), -1) if rot < hd else r

            q, k = rope(q), rope(k)
            if self.k[i] is not None:
                k = torch.cat((self.k[i], k), 2)
                v = torch.cat((self.v[i], v), 2)
            self.k[i], self.v[i] = k, v
            G = Hq // Hkv
            kk, vv = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
            s = (q.float() @ kk.float().transpose(-1, -2)) / math.sqrt(hd)
            L = kk.shape[2]
            qpos = torch.arange(past, past + S, device=self.device)[:, None]
            mask = torch.arange(L, device=self.device)[None] <= qpos
            s = s.masked_fill(~mask, float("-inf"))
            a = (torch.softmax(s, -1) @ vv.float()).to(x.dtype)
            a = a.transpose(1, 2).reshape(B, S, Hq * hd)
            x = x + F.linear(a, sd[p + "self_attn.o_proj.weight"])
            h = self._norm(x, sd[p + "post_attention_layernorm.weight"])
            m = act(F.linear(h, sd[p + "mlp.gate_proj.weight"])) * F.linear(h, sd[p + "mlp.up_proj.weight"])
            x = x + F.linear(m, sd[p + "mlp.down_proj.weight"])
        x = self._norm(x, sd["model.norm.weight"])
        return F.linear(x, sd["lm_head.weight"])

    @torch.no_grad()
    def greedy(self, ids: torch.Tensor, max_new_tokens: int):
        """Returns (tokens [B, n], logits of every generated step [B, n, V])."""
        self.reset()
        logits = self.forward(ids)[:, -1]
        toks, lg = [], []
        for _ in range(max_new_tokens):
            nxt = logits.float().argmax(-1)
            toks.append(nxt)
            lg.append(logits)
            logits = self.forward(nxt[:, None])[:, -1]
        return torch.stack(toks, 1), torch.stack(lg, 1)
