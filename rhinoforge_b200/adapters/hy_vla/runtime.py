"""Hy-Embodied VLA: checkpoint -> :class:`rhinoforge_b200.models.hyvla.HyVlaEngine` with its HYViT2 tower, and the
action-chunk pipeline over a pre-processed observation (``preprocess.build_observation``).

Reference: ``python/rpu_backend/adapters/hy_vla/runtime.py:607-652,821-986`` (pipeline, build),
``adapters/hy_vla/weights.py:425-520`` (position-embedding resampling, weight pick-up).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Optional

import torch
import torch.nn.functional as F

from ...api.errors import RPUBackendError, UnsupportedModelError
from ...models.hyvla import LM_HEAD, MERGER_P, VIT_P, HyVlaConfig, HyVlaEngine, hyvla_shapes


def resample_pos_embedding(pos_embed: torch.Tensor, h: int, w: int) -> torch.Tensor:
    """``[1, n*n, C]`` learned position table -> ``[1, h*w, C]`` sampled bilinearly at the centres of an ``h x w`` grid
    (no corner alignment, border clamped): the table a checkpoint trained at another resolution needs at this one."""
    side = int(round(pos_embed.shape[1] ** 0.5))
    if side * side != pos_embed.shape[1]:
        raise UnsupportedModelError(f"pos_embed holds {pos_embed.shape[1]} rows, not a square grid")
    if (side, side) == (h, w):
        return pos_embed.float()
    table = pos_embed[0].float().t().reshape(1, -1, side, side)
    ys = torch.linspace(-1 + 1.0 / h, 1 - 1.0 / h, h)
    xs = torch.linspace(-1 + 1.0 / w, 1 - 1.0 / w, w)
    gy, gx = torch.meshgrid(ys, xs, indexing="ij")
    grid = torch.stack((gx, gy), -1).reshape(1, h * w, 1, 2)
    out = F.grid_sample(table, grid, mode="bilinear", align_corners=False, padding_mode="border")
    return out.reshape(1, -1, h * w).transpose(1, 2).contiguous()


def build_engine(get_weight: Callable[[str], torch.Tensor], cfg: Optional[HyVlaConfig] = None, *, names=None,
                 prefix_len: int = 240, n_cameras: int = 3, image_size: int = 224, vit_layers: int = 27, vit_heads: int = 16,
                 vit_inter: int = 4304, patch_size: int = 16, device="cuda", dtype=torch.float16) -> HyVlaEngine:
    """Read every tensor both towers, the merger, the head and the HYViT2 tower need and build the engine; refuses
    before any device work when a tensor is missing."""
    from ...models.vision import HYViT2Encoder, SiglipConfig
    cfg = cfg or HyVlaConfig()
    want = [n for n, _, _ in hyvla_shapes(cfg)]
    if names is not None:
        missing = [n for n in want if n not in names]
        if missing:
            raise UnsupportedModelError(f"checkpoint lacks {len(missing)} tensors, first: {missing[0]!r}")
    sd = {n: get_weight(n) for n in want}

    class _Vit(dict):
        def __missing__(_, key):
            t = get_weight(key)
            if key.endswith("pos_embed"):
                side = image_size // patch_size
                t = resample_pos_embedding(t, side, side)
            return t
    vcfg = SiglipConfig(hidden_size=cfg.vit_hidden, intermediate_size=vit_inter, num_hidden_layers=vit_layers,
                        num_attention_heads=vit_heads, image_size=image_size, patch_size=patch_size)
    if (image_size // patch_size) != 2 * cfg.grid:
        raise UnsupportedModelError(f"the tower gives {image_size // patch_size} tokens per side, the merger needs {2 * cfg.grid}")
    tower = HYViT2Encoder(vcfg, _Vit(), prefix=VIT_P, device=device, dtype=dtype, max_images=n_cameras,
                          projector=(sd[MERGER_P + "proj1.weight"], sd[MERGER_P + "proj1.bias"]))
    eng = HyVlaEngine(cfg, sd, max_prefix=prefix_len, device=device, dtype=dtype, vision=tower)
    eng.vision_tower = tower
    return eng


@torch.no_grad()
def get_action(eng: HyVlaEngine, obs: Mapping[str, Any], *, prefix_len: Optional[int] = None, use_graph: bool = True) -> torch.Tensor:
    """One action chunk ``[n_action, action_dim]`` from a pre-processed observation: images -> tower + merger -> prefix
    rows -> twin-weight prefill (cut to the real rows rounded up to 16) -> expert Euler loop."""
    cfg = eng.cfg
    n_valid = int(obs["n_valid"])
    S = min((n_valid + 15) // 16 * 16, int(obs["prefill_pos"].numel()))
    if prefix_len is not None and S > prefix_len:
        raise RPUBackendError(f"the observation has {n_valid} real prefix rows, the policy was built for {prefix_len}")
    images = torch.cat([im.reshape(1, *im.shape[-3:]) for im in obs["images"]], 0)
    embs = eng.embed_images(images)
    rows, vis = eng.build_prefix(list(embs), torch.as_tensor(obs["lang_tokens"]))
    if rows.shape[0] != int(obs["prefill_pos"].numel()) or not torch.equal(vis.cpu(), torch.as_tensor(obs["modality_mask"]).bool().cpu()):
        raise RPUBackendError("the observation's masks do not describe the prefix these images and tokens give")
    eng.prefill(rows[:S], torch.as_tensor(obs["prefill_pos"])[:S], torch.as_tensor(obs["prefill_mask"])[:S, :S], vis[:S])
    L = cfg.suffix_len
    dm = torch.as_tensor(obs["denoise_mask"]).bool()
    dm = torch.cat((dm[:, :S], dm[:, -L:]), 1)
    return eng.denoise(torch.as_tensor(obs["suffix_pos"]), dm, torch.as_tensor(obs["state"], dtype=torch.float32),
                       torch.as_tensor(obs["noise"], dtype=torch.float32), use_graph=use_graph)


__all__ = ["build_engine", "get_action", "resample_pos_embedding"]
