"""Pi0.5 adapter: checkpoint/config mapping for :class:`rhinoforge_b200.api.policy.Pi05Policy`.

A LeRobot Pi0.5 checkpoint directory holds ``config.json`` (policy configuration: chunk size, action
dimension, variant names, image features) and ``model.safetensors`` whose tensors are named
``[model.]paligemma_with_expert.{paligemma,gemma_expert}...``, ``action_in_proj``, ``action_out_proj``,
``time_mlp_in``, ``time_mlp_out``.  This module turns both into a :class:`Pi05Config` and a state dict
with the canonical (prefix-free) names that :mod:`rhinoforge_b200.models.pi05` reads.
Reference: ``python/rpu_backend/adapters/pi05/loader.py``, ``adapters/pi05/__init__.py:315,779-946``.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Tuple

import torch

from ...models.pi05 import GemmaGeometry, Pi05Config
from ...models.vision import SiglipConfig
from ...runtime.errors import UnsupportedModelError

GEMMA_VARIANTS = {
    "gemma_2b": GemmaGeometry(2048, 16384, layers=18, heads=8, kv_heads=1, head_dim=256),
    "gemma_300m": GemmaGeometry(1024, 4096, layers=18, heads=8, kv_heads=1, head_dim=256),
}
ADMITTED = ("gemma_2b", "gemma_300m")


def _get(c, k, d=None):
    return c.get(k, d) if isinstance(c, dict) else getattr(c, k, d)


def config_from_policy_config(pc) -> Tuple[Pi05Config, Dict[str, Any]]:
    """LeRobot ``PI05Config`` (object or its JSON dict) -> (Pi05Config, facade metadata)."""
    vlm, exp = _get(pc, "paligemma_variant", "gemma_2b"), _get(pc, "action_expert_variant", "gemma_300m")
    if (vlm, exp) != ADMITTED:
        raise UnsupportedModelError(f"Pi0.5 variant pair {(vlm, exp)} is not admitted; expected {ADMITTED}")
    if str(_get(pc, "dtype", "float32")) not in ("float32", "bfloat16", "float16"):
        raise UnsupportedModelError("Pi0.5 checkpoint dtype must be float32, bfloat16 or float16")
    res = _get(pc, "image_resolution", (224, 224))
    if tuple(res) != (224, 224):
        raise UnsupportedModelError(f"Pi0.5 image resolution {tuple(res)} is not admitted (224x224 only)")
    feats = _get(pc, "input_features", {}) or {}
    cams = [k for k in feats if k.startswith("observation.images.")]
    out_feats = _get(pc, "output_features", {}) or {}
    act = out_feats.get("action") if isinstance(out_feats, dict) else None
    real_dim = None
    if act is not None:
        shape = _get(act, "shape")
        real_dim = int(shape[0]) if shape else None
    cfg = Pi05Config(vlm=GEMMA_VARIANTS[vlm], expert=GEMMA_VARIANTS[exp], vision=SiglipConfig(),
                     action_dim=int(_get(pc, "max_action_dim", 32)), horizon=int(_get(pc, "chunk_size", 50)),
                     min_period=float(_get(pc, "min_period", 4e-3)), max_period=float(_get(pc, "max_period", 4.0)),
                     max_lang_tokens=int(_get(pc, "tokenizer_max_length", 200)), num_views=max(len(cams), 1) if cams else 3)
    meta = dict(camera_keys=cams or None, n_action_steps=int(_get(pc, "n_action_steps", cfg.horizon)), action_dim=real_dim)
    return cfg, meta


def config_from_lerobot(policy_config, model) -> Tuple[Pi05Config, Dict[str, Any]]:
    if policy_config is None:
        raise UnsupportedModelError("the LeRobot policy carries no config")
    return config_from_policy_config(policy_config)


def canonical_name(name: str) -> str:
    """Strip wrapper prefixes so that names start at ``paligemma_with_expert`` / ``action_*`` / ``time_mlp_*``."""
    for pre in ("model.", "policy.model.", "_orig_mod."):
        if name.startswith(pre):
            name = name[len(pre):]
    # older exports keep the language model one level deeper
    name = name.replace("paligemma.language_model.model.", "paligemma.model.language_model.")
    name = name.replace("paligemma.vision_tower.", "paligemma.model.vision_tower.") \
        if ".paligemma.vision_tower." in name and ".paligemma.model.vision_tower." not in name else name
    name = name.replace("paligemma.multi_modal_projector.", "paligemma.model.multi_modal_projector.") \
        if ".paligemma.multi_modal_projector." in name and ".paligemma.model.multi_modal_projector." not in name else name
    return name


class _LazyStateDict(dict):
    """Tensor access by canonical name, reading from safetensors on demand."""

    def __init__(self, files):
        super().__init__()
        from safetensors import safe_open
        self._where, self._handles = {}, {}
        for f in files:
            h = safe_open(str(f), framework="pt")
            self._handles[str(f)] = h
            for k in h.keys():
                self._where[canonical_name(k)] = (str(f), k)

    def __missing__(self, key):
        if key not in self._where:
            raise KeyError(key)
        f, k = self._where[key]
        return self._handles[f].get_tensor(k)

    def __contains__(self, key):
        return key in self._where

    def __iter__(self):
        return iter(self._where)

    def keys(self):
        return self._where.keys()

    def __len__(self):
        return len(self._where)


def load_checkpoint(path: str):
    """(Pi05Config, state dict view, facade metadata) of a local LeRobot Pi0.5 checkpoint directory.
    Everything is decided from ``config.json`` before a tensor is read."""
    root = Path(path).expanduser()
    cfg_file = root / "config.json"
    if not cfg_file.is_file():
        raise UnsupportedModelError(f"no config.json under {path!r} (a local LeRobot checkpoint directory is required)")
    pc = json.loads(cfg_file.read_text())
    if pc.get("type", "pi05") != "pi05":
        raise UnsupportedModelError(f"checkpoint policy type {pc.get('type')!r} is not pi05")
    cfg, meta = config_from_policy_config(pc)
    # names are canonicalised while reading, so the reference's derived `model_remapped.safetensors` (a cache that can be
    # stale with respect to the shards beside it) is never read
    files = sorted(f for f in root.glob("model*.safetensors") if f.name != "model_remapped.safetensors")
    if not files:
        raise UnsupportedModelError(f"no model*.safetensors under {path!r}")
    return cfg, _LazyStateDict(files), meta


class Pi05Adapter:
    """Kept for symmetry with the other families: ``Pi05Adapter(policy).to_rpu()`` == ``policy.to('rpu')``."""

    def __init__(self, policy, *, rpu_execution=None):
        self.policy = policy
        if rpu_execution is not None:
            policy._rpu_execution = rpu_execution

    @staticmethod
    def preflight(policy_config) -> None:
        config_from_policy_config(policy_config)

    def to_rpu(self, **kw):
        return self.policy.to("rpu", **kw)


__all__ = ["Pi05Adapter", "load_checkpoint", "config_from_lerobot", "config_from_policy_config", "canonical_name"]
