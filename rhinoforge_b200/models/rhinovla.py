"""RhinoVLA action expert: the QwenPI05 layer stack (adaptive RMSNorm, QK norm, prefix K/V, SwiGLU, tanh-gated residual)
behind RhinoVLA's own input / output head and denoise rule.

Per Euler step ``k`` with conditioning row ``c_k`` (the timestep embedding; the same row drives every adaptive norm)::

    a      = action_in_proj(x)                                             # [horizon, W], 72-D actions
    tok    = time_mlp_out(silu(time_mlp_in([a | c_k]))) + action_mask_proj(action_mask)
    state  = state_proj(state) + state_mask_proj(state_mask)               # mask_condition: masks enter as tokens' offsets
    h      = final_norm(expert([state ; tok], c_k))
    v      = action_out_proj(h[1:]) * action_mask
    x      = (x + dt * v) * action_mask                                     # dt = +1 / steps: the schedule runs 0 -> 1

Hoisted: the timestep half of ``time_mlp_in`` (``W[:, W:] c_k + b``) is a per-step bias row, the modulation of every
(step, layer) and of the final norm is the QwenPI05 table, the two mask projections and the state token are computed once
per call.  Instance LoRA deltas are merged into the base weights before the engine is built (:func:`merge_lora`), so the
kernels never see them.  The loop replays from one CUDA graph per step count.

Reference behaviour: ``src/fused/rpu_rhino_vla_model.cpp:1-45`` (expert family, differences from the Pi0.5 expert),
``python/rpu_backend/adapters/rhinovla/convert.py:234-306`` (per-step tables), ``:307-413`` (head weights, padding, folded
time projection), ``python/rpu_backend/adapters/rhinovla/fused.py:1-17`` (LoRA merged before installation).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, Mapping, Optional, Tuple

import torch
import torch.nn.functional as F

from .qwenpi05 import (QwenPI05Config, QwenPI05Engine, TorchQwenPI05, modulation_schedule, qwenpi05_shapes,
                       sinusoidal_embedding)


@dataclass
class RhinoVLAConfig(QwenPI05Config):
    layers: int = 18
    action_dim: int = 72
    state_dim: int = 8
    horizon: int = 30
    num_steps: int = 10


def tiny_rhinovla_config(**kw) -> RhinoVLAConfig:
    base = dict(width=64, layers=3, heads=2, kv_heads=1, head_dim=64, inter=128, rope_theta=1e4, action_dim=9, state_dim=3,
                horizon=6, num_steps=4)
    base.update(kw)
    return RhinoVLAConfig(**base)


def rhinovla_shapes(cfg: RhinoVLAConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    W = cfg.width
    for name, shape, kind in qwenpi05_shapes(cfg):
        if name.startswith("io.time_mlp_"):
            continue
        yield name, shape, kind
    yield "io.action_time_mlp_in.weight", (W, 2 * W), "matrix"
    yield "io.action_time_mlp_in.bias", (W,), "bias"
    yield "io.action_time_mlp_out.weight", (W, W), "matrix"
    yield "io.action_time_mlp_out.bias", (W,), "bias"
    yield "io.state_mask_proj.weight", (W, cfg.state_dim), "matrix"
    yield "io.state_mask_proj.bias", (W,), "bias"
    yield "io.action_mask_proj.weight", (W, cfg.action_dim), "matrix"
    yield "io.action_mask_proj.bias", (W,), "bias"


def random_rhinovla_state_dict(cfg: RhinoVLAConfig, *, seed: int = 0, std: float = 0.05, dtype=torch.float16, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape, kind in rhinovla_shapes(cfg):
        r = torch.randn(shape, generator=g)
        sd[name] = {"matrix": r * std, "norm": 1.0 + 0.05 * r, "bias": 0.03 * r}[kind].to(device, dtype)
    return sd


def merge_lora(base: Mapping[str, torch.Tensor], lora: Mapping[str, torch.Tensor], *, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """``W <- W + scale * B A`` for every ``<name>.lora_A.weight`` / ``<name>.lora_B.weight`` pair (``<name>.weight`` is the
    base matrix); returns a new dict without the LoRA entries."""
    out = {k: v for k, v in base.items()}
    pairs = sorted(k[:-len(".lora_A.weight")] for k in lora if k.endswith(".lora_A.weight"))
    for name in pairs:
        a, b = lora[name + ".lora_A.weight"], lora.get(name + ".lora_B.weight")
        if b is None:
            raise KeyError(f"{name}.lora_B.weight is missing")
        key = name + ".weight"
        if key not in out:
            raise KeyError(f"LoRA pair {name!r} has no base weight {key!r}")
        w = out[key]
        if b.shape[0] != w.shape[0] or a.shape[1] != w.shape[1] or a.shape[0] != b.shape[1]:
            raise ValueError(f"LoRA pair {name!r}: B {tuple(b.shape)} A {tuple(a.shape)} do not produce {tuple(w.shape)}")
        out[key] = (w.float() + float(scale) * (b.float() @ a.float())).to(w.dtype)
    return out


def step_times(num_steps: int):
    """The schedule runs from 0 towards 1 in equal steps."""
    return [k / num_steps for k in range(num_steps)]


def default_cond_table(cfg: RhinoVLAConfig, num_steps: int) -> torch.Tensor:
    """``[num_steps, width]`` fp32 sinusoidal timestep embeddings of :func:`step_times`."""
    return sinusoidal_embedding(torch.tensor(step_times(num_steps)), cfg.width, cfg.min_period, cfg.max_period)


class TorchRhinoVLA(TorchQwenPI05):
    @torch.no_grad()
    def sample_actions(self, prefix_kv, prefix_valid, state, state_mask, noise, action_mask, cond_all: torch.Tensor) -> torch.Tensor:
        cfg, sd, W = self.cfg, self.sd, self.cfg.width
        dev, dt_ = self.device, self.dtype
        steps = cond_all.shape[0]
        x = noise.to(dev, dt_)
        am, sm = action_mask.to(dev, dt_), state_mask.to(dev, dt_).reshape(1, -1)
        n = cfg.suffix_rows
        p0 = int(prefix_valid.long().sum())
        pos = p0 + torch.arange(n, device=dev)
        lin = lambda t, name: F.linear(t, sd[f"io.{name}.weight"], sd[f"io.{name}.bias"])
        st = lin(state.to(dev, dt_).reshape(1, -1), "state_proj") + lin(sm, "state_mask_proj")
        am_tok = lin(am, "action_mask_proj")
        for k in range(steps):
            c = cond_all[k].to(dev, dt_)
            a = lin(x, "action_in_proj")
            tok = lin(F.silu(lin(torch.cat((a, c[None].expand(a.shape[0], -1)), 1), "action_time_mlp_in")), "action_time_mlp_out") + am_tok
            out = self.expert(torch.cat((st, tok), 0), prefix_kv, prefix_valid, torch.ones(n, dtype=torch.bool), pos, c)
            v = lin(out[-cfg.horizon:], "action_out_proj") * am
            x = (x + (1.0 / steps) * v) * am
        return x


class RhinoVLAEngine(QwenPI05Engine):
    def __init__(self, cfg: RhinoVLAConfig, sd: Dict[str, torch.Tensor], **kw):
        if not cfg.use_state_token:
            raise ValueError("the RhinoVLA head always feeds a state token")
        super().__init__(cfg, sd, **kw)
        dev, W = self.device, cfg.width
        self.sd_pad = (cfg.state_dim + 7) // 8 * 8
        z = lambda *s: torch.zeros(*s, dtype=self.dtype, device=dev)
        self.a_emb, self.t_mid, self.v = z(cfg.horizon, W), z(cfg.horizon, W), z(cfg.horizon, self.ad_pad)
        self.amask, self.amask_tok = z(cfg.horizon, self.ad_pad), z(cfg.horizon, W)

    def schedule_for(self, cond_all: torch.Tensor) -> dict:
        cfg, sd, W = self.cfg, self._small, self.cfg.width
        cond = cond_all.to(self.device, torch.float32)
        steps = cond.shape[0]
        key = (steps, hash(cond.cpu().numpy().tobytes()))
        hit = self._schedules.get(key)
        if hit is not None:
            return hit
        mod, fin = modulation_schedule(sd, cfg, cond)
        pad = lambda m, rows, cols: F.pad(m, (0, cols - m.shape[1], 0, rows - m.shape[0]))
        w_in = sd["io.action_time_mlp_in.weight"]
        hit = dict(steps=steps,
                   mod=mod.view(steps, cfg.layers, 2, 1, 3 * W).to(self.dtype).contiguous(), final=fin.to(self.dtype).contiguous(),
                   in_w=pad(sd["io.action_in_proj.weight"], W, self.ad_pad).to(self.dtype).contiguous(),
                   in_b=sd["io.action_in_proj.bias"].to(self.dtype).contiguous(),
                   ta_w=w_in[:, :W].to(self.dtype).contiguous(),
                   t_bias=(F.linear(cond, w_in[:, W:], sd["io.action_time_mlp_in.bias"])).to(self.dtype).contiguous(),   # [steps, W]
                   to_w=sd["io.action_time_mlp_out.weight"].to(self.dtype).contiguous(),
                   to_b=sd["io.action_time_mlp_out.bias"].to(self.dtype).contiguous(),
                   out_w=pad(sd["io.action_out_proj.weight"], self.ad_pad, W).to(self.dtype).contiguous(),
                   out_b=F.pad(sd["io.action_out_proj.bias"], (0, self.ad_pad - cfg.action_dim)).to(self.dtype).contiguous())
        self._schedules[key] = hit
        return hit

    def _rhino_loop(self, sch: dict) -> None:
        cfg, K = self.cfg, self.K
        n, dt = cfg.suffix_rows, 1.0 / sch["steps"]
        for k in range(sch["steps"]):
            K.gemm(self.x, sch["in_w"], bias=sch["in_b"], out=self.a_emb)
            K.gemm(self.a_emb, sch["ta_w"], bias=sch["t_bias"][k], act="silu", out=self.t_mid)
            K.gemm(self.t_mid, sch["to_w"], bias=sch["to_b"], residual=self.amask_tok, out=self.h[1:])
            self.h[0:1].copy_(self.state_emb)
            self._layers(sch["mod"][k])
            K.rmsnorm(self.h, None, cfg.eps, out=self.hn, mod=sch["final"][k:k + 1], rows_per_mod=n)
            K.gemm(self.hn[1:], sch["out_w"], bias=sch["out_b"], out=self.v)
            self.v.mul_(self.amask)
            self.x.add_(self.v, alpha=dt).mul_(self.amask)

    @torch.no_grad()
    def predict(self, state: torch.Tensor, noise: torch.Tensor, *, state_mask: Optional[torch.Tensor] = None,
                action_mask: Optional[torch.Tensor] = None, cond_all: Optional[torch.Tensor] = None,
                num_steps: Optional[int] = None, use_graph: bool = True) -> torch.Tensor:
        """``state [state_dim]``, ``noise [horizon, action_dim]``, masks of the same shapes (default all ones), ``cond_all
        [steps, width]`` (default: sinusoidal embeddings of ``k / steps``) -> ``[horizon, action_dim]`` (an engine buffer)."""
        cfg, dev, sm = self.cfg, self.device, self._small
        if cond_all is None:
            cond_all = default_cond_table(cfg, num_steps or cfg.num_steps)
        sch = self.schedule_for(cond_all)
        f32 = lambda t: t.to(dev, torch.float32)
        state_mask = torch.ones(cfg.state_dim) if state_mask is None else state_mask
        action_mask = torch.ones(cfg.horizon, cfg.action_dim) if action_mask is None else action_mask
        st = F.linear(f32(state).reshape(1, -1), sm["io.state_proj.weight"], sm["io.state_proj.bias"]) \
            + F.linear(f32(state_mask).reshape(1, -1), sm["io.state_mask_proj.weight"], sm["io.state_mask_proj.bias"])
        self.state_emb.copy_(st.to(self.dtype))
        am = f32(action_mask).reshape(cfg.horizon, cfg.action_dim)
        self.amask.zero_()
        self.amask[:, :cfg.action_dim].copy_(am.to(self.dtype))
        self.amask_tok.copy_(F.linear(am, sm["io.action_mask_proj.weight"], sm["io.action_mask_proj.bias"]).to(self.dtype))
        self.x.zero_()
        self.x[:, :cfg.action_dim].copy_(noise.reshape(cfg.horizon, cfg.action_dim).to(dev, self.dtype))
        if not use_graph:
            self._rhino_loop(sch)
        else:
            key = ("rhino", id(sch))
            gph = self._graphs.get(key)
            if gph is None:
                snap = self.x.clone()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._rhino_loop(dict(sch, steps=1))              # warm-up: load kernels, set attributes
                torch.cuda.current_stream().wait_stream(s)
                self.x.copy_(snap)
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph, stream=s):
                    self._rhino_loop(sch)
                torch.cuda.synchronize()
                self.x.copy_(snap)
                self._graphs[key] = gph
            gph.replay()
        return self.x[:, :cfg.action_dim]


__all__ = ["RhinoVLAConfig", "RhinoVLAEngine", "TorchRhinoVLA", "tiny_rhinovla_config", "rhinovla_shapes",
           "random_rhinovla_state_dict", "merge_lora", "default_cond_table", "step_times"]
