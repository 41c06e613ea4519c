"""LingBot-VLA-v2 adapter: checkpoint configuration -> :class:`rhinoforge_b200.models.lingbot2.Lingbot2Engine`.

The checkpoint's ``config.json`` describes the action expert (width, layers, MoE geometry, chunk size, action and state
widths); the Qwen3-VL backbone's configuration comes from its ``vlm_config`` / ``qwen3vl_config`` entry or, when the
checkpoint carries none, from a Qwen3-VL configuration directory given as ``qwen3vl_base``.  All rejections are decided
from the configuration, before a weight is read (reference: ``python/rpu_backend/adapters/lingbot_vla_v2/convert.py:36-160``
for the geometry and tensor names, ``runtime.py:2935-3226`` for the build).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Mapping, Optional

import torch

from ...api.errors import UnsupportedModelError
from ...models.lingbot2 import EXP_P, VLM_P, Lingbot2Config, lingbot2_expert_shapes

# config.json key -> Lingbot2Config field (the names the public checkpoint uses, with this package's names as fallbacks)
_FIELD_KEYS = {
    "hidden": ("expert_hidden_size", "expert_hidden", "hidden"),
    "layers": ("expert_num_hidden_layers", "expert_layers", "layers"),
    "heads": ("expert_num_attention_heads", "heads"),
    "kv_heads": ("expert_num_key_value_heads", "kv_heads"),
    "head_dim": ("expert_head_dim", "head_dim"),
    "eps": ("expert_rms_norm_eps", "rms_norm_eps", "eps"),
    "experts": ("num_experts", "experts"),
    "top_k": ("num_experts_per_tok", "top_k"),
    "routed_inter": ("moe_intermediate_size", "routed_inter"),
    "shared_inter": ("shared_expert_intermediate_size", "shared_inter"),
    "routed_scale": ("routed_scaling_factor", "routed_scale"),
    "horizon": ("chunk_size", "n_action_steps", "horizon"),
    "action_dim": ("max_action_dim", "action_dim"),
    "state_dim": ("max_state_dim", "state_dim"),
    "num_steps": ("num_steps",),
    "blocked_tail": ("blocked_tail",),
}


def expert_config(config: Mapping, rope_theta: float) -> Lingbot2Config:
    src = dict(config.get("expert", {})) if isinstance(config.get("expert"), Mapping) else {}
    src = {**config, **src}
    kw = {}
    for field, keys in _FIELD_KEYS.items():
        for k in keys:
            if k in src and src[k] is not None:
                kw[field] = src[k]
                break
    cfg = Lingbot2Config(rope_theta=rope_theta, **kw)
    preflight(cfg)
    return cfg


def preflight(cfg: Lingbot2Config) -> None:
    """Configuration-only admission: everything the kernels below cannot run is refused here."""
    bad = []
    if cfg.head_dim not in (64, 128, 256):
        bad.append(f"head_dim {cfg.head_dim} (64 / 128 / 256)")
    if cfg.hidden % 8 or cfg.routed_inter % 8 or cfg.shared_inter % 8:
        bad.append("widths that are not multiples of 8")
    if cfg.heads % cfg.kv_heads:
        bad.append(f"{cfg.heads} query heads over {cfg.kv_heads} kv heads")
    if not 0 < cfg.top_k <= cfg.experts or cfg.experts > 256:
        bad.append(f"top-{cfg.top_k} of {cfg.experts} experts")
    if cfg.num_steps < 1 or cfg.horizon < 1:
        bad.append("an empty denoise schedule or action chunk")
    if bad:
        raise UnsupportedModelError("LingBot-VLA-V2 configuration is outside what this framework runs: " + "; ".join(bad))


def _vlm_config(config: Mapping, qwen3vl_base: Optional[str]):
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLConfig
    for key in ("vlm_config", "qwen3vl_config"):
        if isinstance(config.get(key), Mapping):
            return Qwen3VLConfig(**config[key])
    if qwen3vl_base is None:
        raise UnsupportedModelError("the checkpoint's config.json carries no Qwen3-VL configuration (vlm_config); pass "
                                    "qwen3vl_base=<directory with the Qwen3-VL config.json>")
    with open(os.path.join(qwen3vl_base, "config.json"), "r", encoding="utf-8") as f:
        return Qwen3VLConfig(**json.load(f))


def build_engine(config: Mapping, get_weight: Callable[[str], torch.Tensor], *, device="cuda", dtype=torch.float16,
                 max_lang_tokens: int = 72, n_cameras: int = 3, image_size: int = 256, qwen3vl_base: Optional[str] = None):
    from ...models.lingbot2 import Lingbot2Engine
    from ...models.qwen3_vl import text_config_of
    hf = _vlm_config(config, qwen3vl_base)
    theta = float(text_config_of(hf).rope_theta)
    cfg = expert_config(config, theta)
    names = getattr(get_weight, "names", None)
    if names is not None:
        missing = [n for n, _, _ in lingbot2_expert_shapes(cfg) if n not in names]
        if missing:
            raise UnsupportedModelError(f"checkpoint lacks {len(missing)} action-expert tensors, first: {missing[0]!r}")
    vc = hf.vision_config
    per_image = (image_size // vc.patch_size) ** 2
    max_prefix = n_cameras * (per_image // vc.spatial_merge_size ** 2) + max_lang_tokens + cfg.blocked_tail
    return Lingbot2Engine(cfg, hf, get_weight, names=set(names) if names is not None else None, device=device, dtype=dtype,
                          max_prefix=(max_prefix + 15) // 16 * 16, max_patches=n_cameras * per_image)


__all__ = ["build_engine", "expert_config", "preflight", "EXP_P", "VLM_P"]
