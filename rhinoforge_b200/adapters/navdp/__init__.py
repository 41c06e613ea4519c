"""NavDP adapter: the extracted ``navdp_head.safetensors`` of InternVLA-N1 -> :class:`NavdpRuntime`.

NavDP is a standalone diffusion-policy checkpoint, not a ``transformers`` model, so it has a builder of its own instead
of an architecture adapter: ``build_navdp`` reads the tensors, checks them against the fixed 16-layer profile and hands
them to :class:`rhinoforge_b200.models.navdp.NavdpEngine`.  The runtime keeps the reference's two calls -
``predict_noise`` for one step, ``predict_action`` for the 20-step DDPM reverse loop - but runs all sampled trajectories
of a call as one batch and the loop as one CUDA graph.

Reference: ``python/rpu_backend/adapters/navdp/runtime.py:76-140`` (runtime calls), ``:256-330`` (builder and profile check).
"""
from __future__ import annotations

from pathlib import Path
from typing import Mapping, Optional, Union

import torch

from ...models.navdp import NavdpConfig, NavdpEngine, check_state_dict, ddpm_tables
from .._assets import verify_asset_manifest

DEFAULT_SEED = 20260706


class NavdpRuntime:
    def __init__(self, engine: NavdpEngine):
        self.engine, self.cfg = engine, engine.cfg

    @torch.no_grad()
    def predict_noise(self, last_actions: torch.Tensor, timestep, goal_embed: torch.Tensor, rgbd_embed: torch.Tensor) -> torch.Tensor:
        """``eps [B, 32, 3]`` (fp32, on the host) of one decoder pass at ``timestep`` (an int or a one-element tensor)."""
        t = int(torch.as_tensor(timestep).reshape(-1)[0])
        ts, _, _ = ddpm_tables(self.cfg.steps)
        if t not in ts:
            raise ValueError(f"timestep {t} is outside the {self.cfg.steps}-step schedule")
        return self.engine.predict_noise(last_actions, ts.index(t), goal_embed, rgbd_embed)

    @torch.no_grad()
    def predict_action(self, goal_embed: torch.Tensor, rgbd_embed: torch.Tensor, sample_num: int = 4, seed: int = DEFAULT_SEED,
                       init_noise: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``goal_embed [1, 1, 384]``, ``rgbd_embed [1, 32, 384]`` -> actions ``[sample_num, 32, 3]`` fp32 on the host.
        The initial sample and the per-step noise are drawn on the host from ``seed`` (the initial sample first)."""
        cfg = self.cfg
        g = torch.Generator().manual_seed(seed)
        if init_noise is None:
            init_noise = torch.randn(sample_num, cfg.predict_size, cfg.action_dim, generator=torch.Generator().manual_seed(seed))
        b = init_noise.shape[0]
        step_noise = torch.randn(cfg.steps, b, cfg.predict_size, cfg.action_dim, generator=g)
        out = self.engine.predict_action(goal_embed, rgbd_embed, init_noise, step_noise).cpu()
        self.engine.check_status()
        return out

    def destroy(self) -> None:
        self.engine.close()

    close = destroy


def load_navdp_tensors(safetensors_path: Union[str, Path], *, asset_manifest: Optional[Mapping] = None):
    path = Path(safetensors_path).expanduser().resolve()
    verify_asset_manifest((path,), asset_manifest)
    from safetensors.torch import load_file
    return load_file(str(path))


def build_navdp(safetensors_path: Union[str, Path], *, asset_manifest: Optional[Mapping] = None, max_samples: int = 4,
                device="cuda", dtype=torch.float16) -> NavdpRuntime:
    sd = load_navdp_tensors(safetensors_path, asset_manifest=asset_manifest)
    cfg = NavdpConfig()
    layers = {int(k.split(".")[2]) for k in sd if k.startswith("decoder.layers.") and k.split(".")[2].isdigit()}
    if layers != set(range(cfg.layers)):
        raise ValueError(f"NavDP checkpoint has decoder layers {sorted(layers)}; the profile is 0..{cfg.layers - 1}")
    check_state_dict(cfg, sd)
    return NavdpRuntime(NavdpEngine(cfg, sd, max_samples=max_samples, device=device, dtype=dtype))


__all__ = ["NavdpRuntime", "build_navdp", "load_navdp_tensors", "DEFAULT_SEED"]
