"""Logical model aliases -> directories under the local model cache.

Same alias table and resolution rules as the reference
(``python/rpu_backend/model_registry.py:11-88``): an alias maps to a path *relative* to
``RPU_MODEL_CACHE`` (default ``~/.cache/rhinoforge/models``).  Resolving an alias is not a
support claim; admission is decided by the adapter's preflight.  One alias is added here:
``qwen3-32b-w8a16`` for the 32B W8A16 tensor-parallel profile.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Dict

DEFAULT_CACHE_ROOT = Path.home() / ".cache" / "rhinoforge" / "models"

# alias = directory below the cache root, one per line, grouped by kind of model
_ALIAS_TABLE = """
# decoders
qwen3-0.6b = Qwen3-0.6B
qwen3-1.7b = Qwen3-1.7B
qwen3-4b = Qwen3-4B
qwen3-8b = Qwen3-8B
qwen3-14b-w8a16-lmhead-int8 = qwen3_lmhead_int8_ckpts/qwen3-14b-w8a16-lmhead-int8
qwen3-32b-w8a16 = qwen3_lmhead_int8_ckpts/qwen3-32b-w8a16-lmhead-int8
llama-3.2-1b = Llama-3.2-1B
# hybrid
qwen3_5-0.8b = qwen3_5-0.8b
qwen3_5-2b = Qwen3.5-2B
qwen3_5-4b = Qwen3.5-4B
qwen3_5-9b = Qwen3.5-9B
# vl
qwen3-vl-2b = Qwen3-VL-2B-Instruct
qwen3-vl-4b = Qwen3-VL-4B-Instruct
gemma4-e4b = gemma-4-e4b-it
# vision
dinov3-vit-b = dinov3-vitb16-pretrain-lvd1689m
# policies
g05-base = G05/g05-base
pi05-base = pi05_base
pi05-libero-finetuned = pi05_libero_finetuned
pi05-libero-finetuned-w8a16-vlm-expert = pi05_libero_finetuned-w8a16-vlm-expert
pi05-libero-finetuned-w4real-kvint8 = pi05_libero_finetuned-w4real-kvint8
wall-oss-0.5 = wall-oss-0.5
wall-oss-0.5-w8a16 = wall-oss-0.5-w8a16
wall-oss-0.5-w4a16 = wall-oss-0.5-w4a16
wall-oss-0.5-w4a16-pgrp = wall-oss-0.5-w4a16-pgrp
gr00t-n1d7-3b = GR00T-N1.7-3B
lingbot-vla-v2-6b = hf/robbyant/lingbot-vla-v2-6b
internvla-n1-navdp = InternVLA-N1-w-NavDP
hy-embodied-0.5-vla-umi = Hy-Embodied-0.5-VLA-UMI
halo_action_expert = HALO/pytorch_weights_current
"""

MODELS: Dict[str, str] = dict(tuple(part.strip() for part in line.split("=", 1))
                              for line in _ALIAS_TABLE.splitlines() if line.strip() and not line.startswith("#"))


def cache_root() -> Path:
    override = os.environ.get("RPU_MODEL_CACHE")
    return Path(override).expanduser() if override else DEFAULT_CACHE_ROOT


def model_path(name: str) -> Path:
    """Directory of a logical model name; unknown names raise ``KeyError`` listing the known ones."""
    if name not in MODELS:
        raise KeyError(f"Unknown model {name!r}. Known: {', '.join(sorted(MODELS))}")
    return cache_root() / MODELS[name]


def hf_cache_root() -> Path:
    configured = os.environ.get("HF_HOME")
    if configured:
        return Path(configured).expanduser()
    if os.environ.get("RPU_MODEL_CACHE"):
        return cache_root() / ".hf"
    return Path.home() / ".cache" / "huggingface"


def set_hf_home_env() -> None:
    """Route the Hugging Face caches under an explicit ``RPU_MODEL_CACHE``; no-op otherwise."""
    if not os.environ.get("RPU_MODEL_CACHE"):
        return
    root = os.environ.setdefault("HF_HOME", str(hf_cache_root()))
    hub = str(Path(root) / "hub")
    os.environ.setdefault("HF_HUB_CACHE", hub)
    os.environ.setdefault("HUGGINGFACE_HUB_CACHE", hub)
