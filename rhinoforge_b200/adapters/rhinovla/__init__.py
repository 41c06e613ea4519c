"""RhinoVLA adapter: an action-expert module tree with its action head and mask projections (or their state dicts) ->
:class:`rhinoforge_b200.models.rhinovla.RhinoVLAEngine`.

``build_rpu_expert`` flattens the modules into the engine's names (``expert.*`` for the layer stack, ``io.*`` for
``action_in_proj`` / ``state_proj`` / ``action_time_mlp_in`` / ``action_time_mlp_out`` / ``action_out_proj`` and the two
mask projections), merges instance-LoRA deltas into the base matrices first, derives and checks the geometry, and builds
the engine.  The prefix K/V of the language model are handed over per observation with ``engine.set_prefix``.

Reference: ``python/rpu_backend/adapters/rhinovla/runtime.py:8-37`` (builder contract: one expert whose prefix may vary
within ``max_seq_len``), ``adapters/rhinovla/convert.py:307-413`` (head tensors), ``adapters/rhinovla/fused.py:1-17``.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ...api.errors import UnsupportedModelError
from ...models.rhinovla import RhinoVLAConfig, RhinoVLAEngine, merge_lora, rhinovla_shapes


def _sd(obj) -> Dict[str, torch.Tensor]:
    if obj is None:
        return {}
    if isinstance(obj, Mapping):
        return {k: (v.state_dict() if hasattr(v, "state_dict") else v) for k, v in obj.items()} if any(
            hasattr(v, "state_dict") for v in obj.values()) else dict(obj)
    return obj.state_dict()


def expert_state_dict(expert, action_io, mask_proj=None, *, lora: Optional[Mapping[str, torch.Tensor]] = None,
                      lora_scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """Module trees (or plain state dicts) -> the engine's flat names.  ``mask_proj`` maps ``state_mask_proj`` /
    ``action_mask_proj`` to Linear modules (or is a state dict with those prefixes)."""
    out: Dict[str, torch.Tensor] = {}
    for k, v in _sd(expert).items():
        out["expert." + k.replace(".dense.", ".cond.")] = v.detach()
    for k, v in _sd(action_io).items():
        out["io." + k] = v.detach()
    mp = _sd(mask_proj)
    for k, v in mp.items():
        if isinstance(v, Mapping):                       # {"state_mask_proj": module.state_dict(), ...}
            for kk, vv in v.items():
                out[f"io.{k}.{kk}"] = vv.detach()
        else:
            out["io." + k] = v.detach()
    if lora:
        out = merge_lora(out, lora, scale=lora_scale)
    return out


def config_from(sd: Mapping[str, torch.Tensor], *, heads: int, kv_heads: int, horizon: int, **overrides) -> RhinoVLAConfig:
    W = sd["io.action_in_proj.weight"].shape[0]
    layers = len({k.split(".")[2] for k in sd if k.startswith("expert.layers.")})
    q = sd["expert.layers.0.self_attn.q_proj.weight"].shape[0]
    kw = dict(width=W, layers=layers, heads=heads, kv_heads=kv_heads, head_dim=q // heads,
              inter=sd["expert.layers.0.mlp.gate_proj.weight"].shape[0], action_dim=sd["io.action_in_proj.weight"].shape[1],
              state_dim=sd["io.state_proj.weight"].shape[1], horizon=horizon)
    kw.update(overrides)
    return RhinoVLAConfig(**kw)


def preflight(cfg: RhinoVLAConfig, sd: Mapping[str, torch.Tensor]) -> None:
    bad = []
    if cfg.head_dim not in (64, 128, 256):
        bad.append(f"head_dim {cfg.head_dim} (64 / 128 / 256)")
    if cfg.width % 8 or cfg.inter % 8:
        bad.append("widths that are not multiples of 8")
    if cfg.heads % cfg.kv_heads:
        bad.append(f"{cfg.heads} query heads over {cfg.kv_heads} kv heads")
    missing = [n for n, shape, _ in rhinovla_shapes(cfg) if n not in sd or tuple(sd[n].shape) != shape]
    if missing:
        bad.append(f"{len(missing)} tensors missing or of another shape (e.g. {missing[:3]})")
    if bad:
        raise UnsupportedModelError("RhinoVLA expert is outside what this framework runs: " + "; ".join(bad))


def build_rpu_expert(expert, *, action_io, mask_proj, heads: int, kv_heads: int, horizon: int, prefix_len: int = 0,
                     suffix_len: Optional[int] = None, max_seq_len: int = 2048, lora: Optional[Mapping[str, torch.Tensor]] = None,
                     lora_scale: float = 1.0, device="cuda", dtype=torch.float16, **config_overrides) -> RhinoVLAEngine:
    """One engine whose runtime prefix may vary within ``max_seq_len`` (``prefix_len`` is accepted for call compatibility:
    every forward resolves its rows from the prefix handed to ``set_prefix``)."""
    sd = expert_state_dict(expert, action_io, mask_proj, lora=lora, lora_scale=lora_scale)
    cfg = config_from(sd, heads=heads, kv_heads=kv_heads, horizon=horizon, **config_overrides)
    preflight(cfg, sd)
    if suffix_len is not None and suffix_len != cfg.suffix_rows:
        raise ValueError(f"suffix_len {suffix_len} does not match the head's {cfg.suffix_rows} rows (state token + horizon)")
    if prefix_len + cfg.suffix_rows > max_seq_len:
        raise ValueError(f"prefix {prefix_len} + suffix {cfg.suffix_rows} exceed max_seq_len {max_seq_len}")
    return RhinoVLAEngine(cfg, sd, max_prefix=max_seq_len - cfg.suffix_rows, device=device, dtype=dtype)


__all__ = ["build_rpu_expert", "expert_state_dict", "config_from", "preflight"]
