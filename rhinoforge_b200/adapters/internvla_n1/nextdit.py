"""InternVLA-N1 NextDiT adapter: a loaded Lumina NextDiT module (or its state dict) plus the action encoder / decoder
and position table -> :class:`NextDiTRuntime`.

``build_nextdit_runtime`` flattens the modules into the names :class:`rhinoforge_b200.models.nextdit.NextDiTEngine` reads
(``model.*`` for the transformer, ``action_encoder.*``, ``action_decoder.*``, ``action_position``), derives the geometry
from the tensors and checks it.  The runtime keeps the reference's calls: ``denoise_actions`` (a whole Euler schedule as
one graph replay) and ``forward_actions`` (one velocity evaluation); inputs and results are host tensors.

Reference: ``python/rpu_backend/adapters/internvla_n1/nextdit.py:91-126`` (geometry checks), ``:1150-1318`` (runtime
calls), ``:1355-1376`` (builder).
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Mapping, Optional, Sequence, Union

import torch

from ...api.errors import UnsupportedModelError
from ...models.nextdit import NextDiTConfig, NextDiTEngine
from .._assets import verify_asset_manifest

SUPPORTED_FF = (1024, 1536)


def nextdit_state_dict(traj_dit, action_encoder=None, action_decoder=None, action_position: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
    """``traj_dit``: a module whose ``.model`` (or itself) is the Lumina transformer, or a mapping of its tensors with or
    without the ``model.`` prefix."""
    if isinstance(traj_dit, Mapping):
        src = dict(traj_dit)
    else:
        inner = getattr(traj_dit, "model", traj_dit)
        missing = [n for n in ("caption_projection", "time_caption_embed", "layers", "norm_out") if not hasattr(inner, n)]
        if missing:
            raise TypeError(f"not a Lumina NextDiT model; missing {missing}")
        src = {"model." + k: v for k, v in inner.state_dict().items()}
    sd = {}
    for k, v in src.items():
        if not (k.startswith("model.") or k.startswith("action_")):
            k = "model." + k
        sd[k] = v.detach()
    for name, mod in (("action_encoder", action_encoder), ("action_decoder", action_decoder)):
        if mod is not None:
            sd[name + ".weight"], sd[name + ".bias"] = mod.weight.detach(), mod.bias.detach()
    if action_position is not None:
        sd["action_position"] = action_position.detach().reshape(-1, action_position.shape[-1])
    return sd


def config_from(sd: Mapping[str, torch.Tensor], *, heads: int = 6, max_cross_seq_len: int = 320, **overrides) -> NextDiTConfig:
    layers = len({k.split(".")[2] for k in sd if k.startswith("model.layers.")})
    H = sd["model.layers.0.attn1.to_q.weight"].shape[0]
    kw = dict(layers=layers, hidden=H, heads=heads, head_dim=H // heads,
              ff=sd["model.layers.0.feed_forward.linear_1.weight"].shape[0],
              cond_dim=sd["model.caption_projection.weight"].shape[1],
              freq_dim=sd["model.time_caption_embed.timestep_embedder.linear_1.weight"].shape[1],
              action_seq=sd["action_position"].shape[0], action_dim=sd["action_encoder.weight"].shape[1],
              max_cross=max_cross_seq_len)
    kw.update(overrides)
    return NextDiTConfig(**kw)


def preflight(cfg: NextDiTConfig, *, strict: bool = True) -> None:
    bad = []
    if strict and (cfg.layers, cfg.hidden, cfg.heads, cfg.head_dim) != (12, 384, 6, 64):
        bad.append(f"geometry {(cfg.layers, cfg.hidden, cfg.heads, cfg.head_dim)} (the profile is (12, 384, 6, 64))")
    if strict and cfg.ff not in SUPPORTED_FF:
        bad.append(f"feed-forward width {cfg.ff} (one of {SUPPORTED_FF})")
    if cfg.heads * cfg.head_dim != cfg.hidden or cfg.head_dim not in (64, 128, 256):
        bad.append(f"{cfg.heads} heads of {cfg.head_dim} over width {cfg.hidden}")
    if bad:
        raise UnsupportedModelError("InternVLA-N1 NextDiT is outside what this framework runs: " + "; ".join(bad))


class NextDiTRuntime:
    def __init__(self, engine: NextDiTEngine):
        self.engine, self.cfg = engine, engine.cfg

    def _check(self, actions: torch.Tensor, condition: torch.Tensor) -> None:
        c = self.cfg
        if actions.dim() != 3 or tuple(actions.shape[1:]) != (c.action_seq, c.action_dim) or not 1 <= actions.shape[0] <= c.max_batch:
            raise ValueError(f"actions must be [B, {c.action_seq}, {c.action_dim}] with B in [1, {c.max_batch}]")
        if condition.dim() != 3 or condition.shape[0] != 1:
            raise ValueError("condition must be [1, S, C]: one condition shared by the trajectories of a call")

    @torch.no_grad()
    def denoise_actions(self, actions: torch.Tensor, timesteps: torch.Tensor, euler_steps: torch.Tensor, condition: torch.Tensor, *,
                        reuse_condition: bool = True) -> torch.Tensor:
        self._check(actions, condition)
        out = self.engine.denoise_actions(actions, timesteps, euler_steps, condition, reuse_condition=reuse_condition).cpu()
        self.engine.check_status()
        return out

    @torch.no_grad()
    def forward_actions(self, actions: torch.Tensor, timestep: torch.Tensor, condition: torch.Tensor) -> torch.Tensor:
        """The model's raw update at one timestep: ``denoise_actions`` with a unit step minus its input."""
        self._check(actions, condition)
        out = self.engine.denoise_actions(actions, timestep.reshape(1), torch.ones(1), condition).cpu()
        self.engine.check_status()
        return out - actions.float()

    def destroy(self) -> None:
        self.engine.close()

    close = destroy


def build_nextdit_runtime(traj_dit, *, max_cross_seq_len: int = 320, action_encoder=None, action_decoder=None,
                          action_position: Optional[torch.Tensor] = None, asset_manifest: Optional[Mapping] = None,
                          asset_paths: Optional[Sequence[Union[str, Path]]] = None, heads: int = 6, strict: bool = True,
                          device="cuda", dtype=torch.float16) -> NextDiTRuntime:
    if asset_manifest is not None:
        verify_asset_manifest(tuple(asset_paths or ()), asset_manifest)
    sd = nextdit_state_dict(traj_dit, action_encoder, action_decoder, action_position)
    for need in ("action_encoder.weight", "action_decoder.weight", "action_position"):
        if need not in sd:
            raise ValueError(f"the runtime integrates actions on the device and needs `{need.split('.')[0]}`")
    cfg = config_from(sd, heads=heads, max_cross_seq_len=max_cross_seq_len)
    preflight(cfg, strict=strict)
    return NextDiTRuntime(NextDiTEngine(cfg, sd, device=device, dtype=dtype))


__all__ = ["NextDiTRuntime", "build_nextdit_runtime", "nextdit_state_dict", "config_from", "preflight"]
