"""QwenPI05 adapter: an action-expert module tree (or its state dict) -> :class:`rhinoforge_b200.models.qwenpi05.QwenPI05Engine`.

The expert arrives as a PyTorch module with ``layers[i].self_attn.{q,k,v,o}_proj``, ``self_attn.{q,k}_norm``,
``mlp.{gate,up,down}_proj`` and adaptive norms ``input_layernorm`` / ``post_attention_layernorm`` / ``norm`` that each
hold ``norm.weight`` and a ``cond`` Linear (older checkpoints call it ``dense``), plus an input / output head with
``action_in_proj``, ``state_proj``, ``time_mlp_in``, ``time_mlp_out`` and ``action_out_proj``.  ``expert_state_dict``
flattens both into the names the engine reads; ``build_engine`` checks the geometry first.

Reference: ``python/rpu_backend/adapters/qwenpi05/fused.py:118-330,538-680`` (weight gathering, install),
``adapters/qwenpi05/convert.py:112-204`` (module conversion).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ...api.errors import UnsupportedModelError
from ...models.qwenpi05 import QwenPI05Config, qwenpi05_shapes


def expert_state_dict(expert_sd: Mapping[str, torch.Tensor], io_sd: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """``expert.*`` / ``io.*`` names out of the two modules' own state dicts (``dense`` is accepted for ``cond``)."""
    out = {}
    for k, v in expert_sd.items():
        out["expert." + k.replace(".dense.", ".cond.")] = v
    for k, v in io_sd.items():
        out["io." + k] = v
    return out


def config_from(expert_config, io_config=None, **overrides) -> QwenPI05Config:
    g = lambda o, k, d=None: (o.get(k, d) if isinstance(o, Mapping) else getattr(o, k, d)) if o is not None else d
    kw = dict(width=g(expert_config, "width"), layers=g(expert_config, "num_hidden_layers", g(expert_config, "depth")),
              heads=g(expert_config, "num_attention_heads"), kv_heads=g(expert_config, "num_key_value_heads"),
              head_dim=g(expert_config, "head_dim"), inter=g(expert_config, "intermediate_size", g(expert_config, "mlp_dim")),
              eps=g(expert_config, "rms_norm_eps", 1e-6), rope_theta=g(expert_config, "rope_theta", 5e6),
              action_dim=g(io_config, "action_dim", 32), state_dim=g(io_config, "state_dim", 32),
              horizon=g(io_config, "action_horizon", 30))
    kw = {k: v for k, v in kw.items() if v is not None}
    kw.update(overrides)
    cfg = QwenPI05Config(**kw)
    preflight(cfg)
    return cfg


def preflight(cfg: QwenPI05Config) -> None:
    bad = []
    if cfg.head_dim not in (64, 128, 256):
        bad.append(f"head_dim {cfg.head_dim} (64 / 128 / 256)")
    if cfg.width % 8 or cfg.inter % 8:
        bad.append("widths that are not multiples of 8")
    if cfg.heads % cfg.kv_heads:
        bad.append(f"{cfg.heads} query heads over {cfg.kv_heads} kv heads")
    if cfg.horizon < 1 or cfg.num_steps < 1:
        bad.append("an empty action chunk or denoise schedule")
    if bad:
        raise UnsupportedModelError("QwenPI05 configuration is outside what this framework runs: " + "; ".join(bad))


def build_engine(cfg: QwenPI05Config, sd: Mapping[str, torch.Tensor], *, max_prefix: int = 1024, device="cuda",
                 dtype=torch.float16):
    from ...models.qwenpi05 import QwenPI05Engine
    preflight(cfg)
    missing = [n for n, shape, _ in qwenpi05_shapes(cfg) if n not in sd]
    if missing:
        raise UnsupportedModelError(f"state dict lacks {len(missing)} expert tensors, first: {missing[0]!r}")
    wrong = [(n, tuple(sd[n].shape), shape) for n, shape, _ in qwenpi05_shapes(cfg) if tuple(sd[n].shape) != shape]
    if wrong:
        n, got, want = wrong[0]
        raise UnsupportedModelError(f"{n!r} has shape {got}, the configuration needs {want}")
    return QwenPI05Engine(cfg, dict(sd), max_prefix=max_prefix, device=device, dtype=dtype)


__all__ = ["build_engine", "config_from", "expert_state_dict", "preflight"]
