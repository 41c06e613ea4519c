"""QwenPI05 action expert: a flow-matching transformer that reads a Qwen3-VL prefix's keys and values.

The expert is the Pi0.5 action-expert recipe on Qwen3 building blocks: adaptive RMSNorm (a learned RMSNorm weight, then
``* (1 + scale) + shift`` with ``[scale | shift | gate] = cond_linear(c)`` of the time conditioning ``c``), per-head
QK RMSNorm, rotary embedding at text-like positions (all three M-RoPE axes equal, so plain 1-D RoPE), grouped-query
attention over ``[prefix K/V of decoder layers offset .. offset + L) | suffix rows]`` under a padding-aware
bidirectional mask, SwiGLU MLP, and a **tanh-gated** residual ``h <- h + tanh(gate) * sublayer(h)``.

Everything that depends on the time step only is hoisted out of the layers: for every (step, layer, norm) the row
``[gamma * (1 + scale) - 1 | shift | tanh(gate)]`` is what the stack's modulated RMSNorm and gated residual consume, so
the learned norm weight and the tanh cost nothing at run time.  The Euler loop (``t = 1 -> 0``, ``dt = -1 / steps``)
replays from one CUDA graph.

The action input / output head here is the Pi0.5-style one (state token, ``action_in_proj``, a two-layer swish time MLP
producing the conditioning, ``action_out_proj``); an application with its own head calls :meth:`QwenPI05Engine.forward`
with its own suffix rows and conditioning.

Reference behaviour: ``src/fused/rpu_qwenpi05_model.cpp:1-40,785-840`` (recipe, tanh-gated residual),
``python/rpu_backend/adapters/qwenpi05/fused.py:29-64,252-330,677-780`` (AdaRMSNorm, weights, M-RoPE of the suffix, mask),
``adapters/qwenpi05/convert.py:206-339`` (one step, the denoise loop).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass
class QwenPI05Config:
    width: int = 1024
    layers: int = 10
    heads: int = 16
    kv_heads: int = 8
    head_dim: int = 128
    inter: int = 4096
    eps: float = 1e-6
    rope_theta: float = 5e6
    action_dim: int = 32
    state_dim: int = 32
    horizon: int = 30
    num_steps: int = 10
    prefix_layer_offset: int = 0     # first prefix-decoder layer whose K/V expert layer 0 reads
    use_state_token: bool = True
    min_period: float = 4e-3
    max_period: float = 4.0

    @property
    def suffix_rows(self) -> int:
        return self.horizon + (1 if self.use_state_token else 0)


def tiny_qwenpi05_config(**kw) -> QwenPI05Config:
    base = dict(width=64, layers=3, heads=2, kv_heads=1, head_dim=64, inter=128, rope_theta=1e4, action_dim=7, state_dim=5,
                horizon=6, num_steps=4)
    base.update(kw)
    return QwenPI05Config(**base)


def qwenpi05_shapes(cfg: QwenPI05Config) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    W, hd = cfg.width, cfg.head_dim
    for i in range(cfg.layers):
        b = f"expert.layers.{i}."
        yield b + "self_attn.q_proj.weight", (cfg.heads * hd, W), "matrix"
        yield b + "self_attn.k_proj.weight", (cfg.kv_heads * hd, W), "matrix"
        yield b + "self_attn.v_proj.weight", (cfg.kv_heads * hd, W), "matrix"
        yield b + "self_attn.o_proj.weight", (W, cfg.heads * hd), "matrix"
        yield b + "self_attn.q_norm.weight", (hd,), "norm"
        yield b + "self_attn.k_norm.weight", (hd,), "norm"
        yield b + "mlp.gate_proj.weight", (cfg.inter, W), "matrix"
        yield b + "mlp.up_proj.weight", (cfg.inter, W), "matrix"
        yield b + "mlp.down_proj.weight", (W, cfg.inter), "matrix"
        for n in ("input_layernorm", "post_attention_layernorm"):
            yield b + n + ".norm.weight", (W,), "norm"
            yield b + n + ".cond.weight", (3 * W, W), "matrix"
            yield b + n + ".cond.bias", (3 * W,), "bias"
    yield "expert.norm.norm.weight", (W,), "norm"
    yield "expert.norm.cond.weight", (3 * W, W), "matrix"
    yield "expert.norm.cond.bias", (3 * W,), "bias"
    yield "io.action_in_proj.weight", (W, cfg.action_dim), "matrix"
    yield "io.action_in_proj.bias", (W,), "bias"
    yield "io.state_proj.weight", (W, cfg.state_dim), "matrix"
    yield "io.state_proj.bias", (W,), "bias"
    yield "io.time_mlp_in.weight", (W, W), "matrix"
    yield "io.time_mlp_in.bias", (W,), "bias"
    yield "io.time_mlp_out.weight", (W, W), "matrix"
    yield "io.time_mlp_out.bias", (W,), "bias"
    yield "io.action_out_proj.weight", (cfg.action_dim, W), "matrix"
    yield "io.action_out_proj.bias", (cfg.action_dim,), "bias"


def random_qwenpi05_state_dict(cfg: QwenPI05Config, *, seed: int = 0, std: float = 0.05, dtype=torch.float16,
                               device="cpu") -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in qwenpi05_shapes(cfg):
        r = torch.randn(shape, generator=g)
        sd[name] = {"matrix": r * std, "norm": 1.0 + 0.05 * r, "bias": 0.03 * r}[kind].to(device, dtype)
    return sd


def sinusoidal_embedding(t: torch.Tensor, dim: int, min_period: float, max_period: float) -> torch.Tensor:
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float32)
    period = min_period * (max_period / min_period) ** frac
    ang = (2.0 * math.pi / period)[None, :] * t.float()[:, None]
    return torch.cat((ang.sin(), ang.cos()), 1)


def euler_times(num_steps: int) -> List[float]:
    out, t = [], 1.0
    for _ in range(num_steps):
        out.append(t)
        t = max(t - 1.0 / num_steps, 0.0)
    return out


def time_conditioning(sd: Dict[str, torch.Tensor], cfg: QwenPI05Config, num_steps: int) -> torch.Tensor:
    """``[num_steps, width]`` fp32: ``swish(W2 swish(W1 sincos(t_k)))``."""
    emb = sinusoidal_embedding(torch.tensor(euler_times(num_steps)), cfg.width, cfg.min_period, cfg.max_period)
    emb = emb.to(sd["io.time_mlp_in.weight"].device)
    h = F.silu(F.linear(emb, sd["io.time_mlp_in.weight"].float(), sd["io.time_mlp_in.bias"].float()))
    return F.silu(F.linear(h, sd["io.time_mlp_out.weight"].float(), sd["io.time_mlp_out.bias"].float()))


def suffix_mask_matrix(prefix_valid: torch.Tensor, suffix_valid: torch.Tensor, width: int) -> torch.Tensor:
    """Boolean ``[n, width]``: every suffix row attends to the valid prefix rows and to the valid suffix rows (cache row =
    prefix rows first, suffix rows behind them); a padded suffix row still sees itself so its softmax is defined."""
    P, n = int(prefix_valid.numel()), int(suffix_valid.numel())
    m = torch.zeros(n, width, dtype=torch.bool)
    m[:, :P] = prefix_valid.bool()[None]
    m[:, P:P + n] = suffix_valid.bool()[None]
    idx = torch.arange(n)
    m[idx, P + idx] = True
    return m


def modulation_schedule(sd: Dict[str, torch.Tensor], cfg: QwenPI05Config, cond: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(mod [steps, layers, 2, 3W], final [steps, 3W])`` fp32 rows ``[gamma * (1 + scale) - 1 | shift | tanh(gate)]``
    for the stack's ``norm(h) * (1 + .) + .`` and ``h += gate * sublayer``."""
    W = cfg.width

    def rows(p: str) -> torch.Tensor:
        m = F.linear(cond, sd[p + ".cond.weight"].float(), sd[p + ".cond.bias"].float())
        gamma = sd[p + ".norm.weight"].float()
        return torch.cat((gamma * (1.0 + m[:, :W]) - 1.0, m[:, W:2 * W], torch.tanh(m[:, 2 * W:])), -1)
    mods = [torch.stack([rows(f"expert.layers.{i}.{n}") for n in ("input_layernorm", "post_attention_layernorm")], 1)
            for i in range(cfg.layers)]
    return torch.stack(mods, 1), rows("expert.norm")


# ----------------------------------------------------------------------------- fp32 oracle
class TorchQwenPI05:
    """Plain PyTorch statement of the expert and the denoise loop (no hoisting, no folds)."""

    def __init__(self, cfg: QwenPI05Config, sd: Dict[str, torch.Tensor], *, dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.sd = {k: v.to(self.device, dtype) for k, v in sd.items()}

    def _rms(self, t, w=None):
        tf = t.float()
        y = tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + self.cfg.eps)
        return y if w is None else y * w.float()

    def _rope(self, t, pos):      # t [heads, n, hd]
        cfg = self.cfg
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32, device=self.device) / cfg.head_dim))
        ang = pos.float()[None, :, None] * inv
        cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)
        h = t.shape[-1] // 2
        return (t.float() * cos + torch.cat((-t[..., h:], t[..., :h]), -1).float() * sin).to(t.dtype)

    def _ada(self, p: str, h, c):
        W = self.cfg.width
        m = F.linear(c, self.sd[p + ".cond.weight"], self.sd[p + ".cond.bias"]).float()
        y = self._rms(h, self.sd[p + ".norm.weight"]) * (1.0 + m[:W]) + m[W:2 * W]
        return y.to(self.dtype), m[2 * W:]

    @torch.no_grad()
    def expert(self, h, prefix_kv, prefix_valid, suffix_valid, pos, c) -> torch.Tensor:
        """``h [n, W]`` suffix rows, ``c [W]`` conditioning -> final-normed hidden ``[n, W]``."""
        cfg, sd = self.cfg, self.sd
        n, hd, G = h.shape[0], cfg.head_dim, cfg.heads // cfg.kv_heads
        P = int(prefix_valid.numel())
        mask = suffix_mask_matrix(prefix_valid, suffix_valid, P + n).to(self.device)
        for i in range(cfg.layers):
            b = f"expert.layers.{i}."
            y, gate = self._ada(b + "input_layernorm", h, c)
            q = F.linear(y, sd[b + "self_attn.q_proj.weight"]).view(n, cfg.heads, hd)
            k = F.linear(y, sd[b + "self_attn.k_proj.weight"]).view(n, cfg.kv_heads, hd)
            v = F.linear(y, sd[b + "self_attn.v_proj.weight"]).view(n, cfg.kv_heads, hd).transpose(0, 1)
            q = self._rms(q, sd[b + "self_attn.q_norm.weight"]).to(self.dtype).transpose(0, 1)
            k = self._rms(k, sd[b + "self_attn.k_norm.weight"]).to(self.dtype).transpose(0, 1)
            q, k = self._rope(q, pos), self._rope(k, pos)
            pk, pv = prefix_kv[cfg.prefix_layer_offset + i]
            ka = torch.cat((pk.to(self.device, self.dtype), k), 1).repeat_interleave(G, 0)
            va = torch.cat((pv.to(self.device, self.dtype), v), 1).repeat_interleave(G, 0)
            s = (q.float() @ ka.float().transpose(-1, -2)) / math.sqrt(hd)
            s = s.masked_fill(~mask[None], float("-inf"))
            o = (torch.softmax(s, -1) @ va.float()).to(self.dtype).transpose(0, 1).reshape(n, -1)
            h = h + (torch.tanh(gate) * F.linear(o, sd[b + "self_attn.o_proj.weight"]).float()).to(self.dtype)
            y, gate = self._ada(b + "post_attention_layernorm", h, c)
            m = F.linear(F.silu(F.linear(y, sd[b + "mlp.gate_proj.weight"])) * F.linear(y, sd[b + "mlp.up_proj.weight"]),
                         sd[b + "mlp.down_proj.weight"])
            h = h + (torch.tanh(gate) * m.float()).to(self.dtype)
        return self._ada("expert.norm", h, c)[0]

    @torch.no_grad()
    def sample_actions(self, prefix_kv, prefix_valid: torch.Tensor, state: Optional[torch.Tensor], noise: torch.Tensor,
                       num_steps: Optional[int] = None) -> torch.Tensor:
        cfg, sd = self.cfg, self.sd
        num_steps = num_steps or cfg.num_steps
        x = noise.to(self.device, self.dtype)
        n = cfg.suffix_rows
        valid = torch.ones(n, dtype=torch.bool)
        p0 = int(prefix_valid.long().sum())
        pos = p0 + torch.arange(n, device=self.device)
        dt = -1.0 / num_steps
        for t in euler_times(num_steps):
            emb = sinusoidal_embedding(torch.tensor([t]), cfg.width, cfg.min_period, cfg.max_period).to(self.device, self.dtype)
            c = F.silu(F.linear(F.silu(F.linear(emb, sd["io.time_mlp_in.weight"], sd["io.time_mlp_in.bias"])),
                                sd["io.time_mlp_out.weight"], sd["io.time_mlp_out.bias"]))[0]
            rows = [F.linear(x, sd["io.action_in_proj.weight"], sd["io.action_in_proj.bias"])]
            if cfg.use_state_token:
                rows.insert(0, F.linear(state.to(self.device, self.dtype).reshape(1, -1), sd["io.state_proj.weight"],
                                        sd["io.state_proj.bias"]))
            out = self.expert(torch.cat(rows, 0), prefix_kv, prefix_valid, valid, pos, c)
            v = F.linear(out[-cfg.horizon:], sd["io.action_out_proj.weight"], sd["io.action_out_proj.bias"])
            x = x + dt * v
        return x


# ----------------------------------------------------------------------------- device engine
class QwenPI05Engine:
    """The expert on the accelerator over a paged KV cache whose prefix rows come from outside (:meth:`set_prefix`).

    ``predict(state, noise)`` runs the whole denoise loop; ``forward(suffix_rows, cond)`` is one expert pass for
    applications with their own input / output head."""

    def __init__(self, cfg: QwenPI05Config, sd: Dict[str, torch.Tensor], *, max_prefix: int = 1024, device="cuda",
                 dtype=torch.float16):
        from ..ops import kernels as K
        from ..runtime.kv_cache import PagedKV
        from ..runtime.stack import NativeStack, StackSpec
        self.K, self.cfg, self.device, self.dtype = K, cfg, torch.device(device), dtype
        dev, n, W = self.device, cfg.suffix_rows, cfg.width
        self.max_prefix = max_prefix
        self.max_seq = (max_prefix + n + 15) // 16 * 16
        self.cache = PagedKV(cfg.layers, 1, self.max_seq, cfg.kv_heads, cfg.head_dim, device=device, dtype=dtype)
        self.cache.reserve_all()
        g = lambda k: sd[k]
        layers = []
        for i in range(cfg.layers):
            b = f"expert.layers.{i}."
            layers.append(dict(
                wqkv=torch.cat([g(b + f"self_attn.{x}_proj.weight") for x in "qkv"], 0), wo=g(b + "self_attn.o_proj.weight"),
                q_norm_w=g(b + "self_attn.q_norm.weight"), k_norm_w=g(b + "self_attn.k_norm.weight"),
                w_up=torch.cat((g(b + "mlp.gate_proj.weight"), g(b + "mlp.up_proj.weight")), 0),
                w_down=g(b + "mlp.down_proj.weight")))
        self.rows = (n + 15) // 16 * 16
        self.stack = NativeStack(
            StackSpec(layers=cfg.layers, hidden=W, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
                      inter=cfg.inter, norm="adarms", mlp="swiglu", eps=cfg.eps, qk_norm=True, rot_dim=cfg.head_dim,
                      gated_residual=True, paged_kv=True, causal=False, max_tokens=self.rows, max_seqs=1),
            layers, device=device, dtype=dtype, kv_cache=self.cache)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32) / cfg.head_dim))
        ang = torch.arange(self.max_seq + 64, dtype=torch.float32)[:, None] * inv[None]
        self.cos, self.sin = ang.cos().to(dev).contiguous(), ang.sin().to(dev).contiguous()
        self._small = {k: v.to(dev, torch.float32) for k, v in sd.items()
                       if k.startswith("io.") or ".cond." in k or ".norm.weight" in k}
        self.ad_pad = (cfg.action_dim + 7) // 8 * 8
        self._schedules: Dict[int, dict] = {}
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        i32 = dict(dtype=torch.int32, device=dev)
        self.x = torch.zeros(cfg.horizon, self.ad_pad, dtype=dtype, device=dev)
        self.h = torch.zeros(n, W, dtype=dtype, device=dev)
        self.hn = torch.zeros(n, W, dtype=dtype, device=dev)
        self.state_emb = torch.zeros(1, W, dtype=dtype, device=dev)
        self.s_pos = torch.zeros(n, **i32)
        self.s_cache_pos = torch.zeros(n, **i32)
        self.s_seq = torch.zeros(n, **i32)
        self.s_qstart = torch.zeros(1, **i32)
        self.s_qlen = torch.full((1,), n, **i32)
        self.s_kvlen = torch.zeros(1, **i32)
        # row pitch a multiple of the attention kernel's 128-key block: its 16-byte mask loads then never cross a row end
        self.mask = torch.zeros(n, (self.max_seq + 127) // 128 * 128, dtype=torch.uint8, device=dev)[:, :self.max_seq]
        self.prefix_len = 0

    # ------------------------------------------------------------------ prefix
    @torch.no_grad()
    def set_prefix(self, prefix_kv: Sequence[Tuple[torch.Tensor, torch.Tensor]], prefix_valid: Optional[torch.Tensor] = None) -> int:
        """Copy the prefix decoder's rotated keys / values (``[kv_heads, P, head_dim]`` per layer; layers
        ``prefix_layer_offset ..`` are used) into the cache and set the positions, lengths and mask of the suffix rows."""
        cfg, dev, n = self.cfg, self.device, self.cfg.suffix_rows
        P = int(prefix_kv[cfg.prefix_layer_offset][0].shape[1])
        if P > self.max_prefix:
            raise ValueError(f"prefix of {P} rows exceeds max_prefix {self.max_prefix}")
        if len(prefix_kv) < cfg.prefix_layer_offset + cfg.layers:
            raise ValueError(f"need prefix K/V of layers [{cfg.prefix_layer_offset}, {cfg.prefix_layer_offset + cfg.layers}), "
                             f"got {len(prefix_kv)} layers")
        valid = torch.ones(P, dtype=torch.bool) if prefix_valid is None else prefix_valid.flatten().bool().cpu()
        for i in range(cfg.layers):
            k, v = prefix_kv[cfg.prefix_layer_offset + i]
            self.cache.scatter(i, 0, k, v, 0)
        self.cache.sync_table()
        p0 = int(valid.long().sum())
        ar = torch.arange(n, dtype=torch.int32)
        self.s_pos.copy_((ar + p0).to(dev))
        self.s_cache_pos.copy_((ar + P).to(dev))
        self.s_kvlen.fill_(P + n)
        self.mask.copy_(suffix_mask_matrix(valid, torch.ones(n, dtype=torch.bool), self.max_seq).to(torch.uint8).to(dev))
        self.prefix_len = P
        return P

    # ------------------------------------------------------------------ schedule
    def schedule(self, num_steps: int) -> dict:
        hit = self._schedules.get(num_steps)
        if hit is not None:
            return hit
        cfg, sd = self.cfg, self._small
        cond = time_conditioning(sd, cfg, num_steps)
        mod, fin = modulation_schedule(sd, cfg, cond)
        dt = -1.0 / num_steps
        pad = lambda m, rows, cols: F.pad(m, (0, cols - m.shape[1], 0, rows - m.shape[0]))
        hit = dict(mod=mod.view(num_steps, cfg.layers, 2, 1, 3 * cfg.width).to(self.dtype).contiguous(),
                   final=fin.to(self.dtype).contiguous(),
                   in_w=pad(sd["io.action_in_proj.weight"], cfg.width, self.ad_pad).to(self.dtype).contiguous(),
                   in_b=sd["io.action_in_proj.bias"].to(self.dtype).contiguous(),
                   out_w=pad(sd["io.action_out_proj.weight"] * dt, self.ad_pad, cfg.width).to(self.dtype).contiguous(),
                   out_b=F.pad(sd["io.action_out_proj.bias"] * dt, (0, self.ad_pad - cfg.action_dim)).to(self.dtype).contiguous())
        self._schedules[num_steps] = hit
        return hit

    # ------------------------------------------------------------------ one pass / the loop
    def _layers(self, mod: torch.Tensor) -> None:
        n = self.cfg.suffix_rows
        self.stack.forward(self.h, q_start=self.s_qstart, q_len=self.s_qlen, kv_len=self.s_kvlen, max_q_len=n,
                           max_kv_len=self.max_seq, pos=self.s_pos, cos=self.cos, sin=self.sin, seq_of_tok=self.s_seq,
                           cache_pos=self.s_cache_pos, page_table=self.cache.page_table, mask=self.mask, mod=mod,
                           rows_per_mod=n)

    @torch.no_grad()
    def forward(self, suffix_rows: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        """One expert pass over given suffix rows ``[suffix_rows, width]`` and conditioning ``[width]``: the final
        modulated-normed hidden rows (a buffer the next call overwrites)."""
        cfg, sd = self.cfg, self._small
        mod, fin = modulation_schedule(sd, cfg, cond.to(self.device, torch.float32).reshape(1, -1))
        self.h.copy_(suffix_rows.to(self.device, self.dtype))
        self._layers(mod.view(cfg.layers, 2, 1, 3 * cfg.width).to(self.dtype).contiguous())
        self.K.rmsnorm(self.h, None, cfg.eps, out=self.hn, mod=fin.to(self.dtype).contiguous(), rows_per_mod=cfg.suffix_rows)
        return self.hn

    def _denoise_loop(self, num_steps: int) -> None:
        cfg, K, sch = self.cfg, self.K, self.schedule(num_steps)
        n, s0 = cfg.suffix_rows, cfg.suffix_rows - cfg.horizon
        for k in range(num_steps):
            K.gemm(self.x, sch["in_w"], bias=sch["in_b"], out=self.h[s0:])
            if s0:
                self.h[0:1].copy_(self.state_emb)
            self._layers(sch["mod"][k])
            K.rmsnorm(self.h, None, cfg.eps, out=self.hn, mod=sch["final"][k:k + 1], rows_per_mod=n)
            K.gemm(self.hn[s0:], sch["out_w"], bias=sch["out_b"], residual=self.x, out=self.x)     # x <- x + dt * v

    @torch.no_grad()
    def predict(self, state: Optional[torch.Tensor], noise: torch.Tensor, num_steps: Optional[int] = None, *,
                use_graph: bool = True) -> torch.Tensor:
        """The denoise loop over the current prefix: ``[horizon, action_dim]`` (a buffer the next call overwrites)."""
        cfg, dev = self.cfg, self.device
        num_steps = num_steps or cfg.num_steps
        if cfg.use_state_token:
            if state is None:
                raise ValueError("this expert reads a state token: pass state")
            st = F.linear(state.to(dev, torch.float32).reshape(1, -1), self._small["io.state_proj.weight"],
                          self._small["io.state_proj.bias"])
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
        self.stack.check_status()

    def close(self) -> None:
        self._graphs.clear()
        self.stack.close()
        self.cache.close()


__all__ = ["QwenPI05Config", "QwenPI05Engine", "TorchQwenPI05", "tiny_qwenpi05_config", "qwenpi05_shapes",
           "random_qwenpi05_state_dict", "modulation_schedule", "time_conditioning", "suffix_mask_matrix", "euler_times"]
