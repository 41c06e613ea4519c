"""Checks shared by the public ``from_pretrained`` entry points: target device, architecture
routing, checkpoint tensor access (reference: ``python/rpu_backend/api/_loading.py:25-79``)."""
from __future__ import annotations

import json
from collections.abc import Collection
from pathlib import Path
from typing import Callable, Dict

import torch

from .errors import UnsupportedModelError

_ROUTES = {
    "DINOv3ViTModel": "use DINOv3Adapter with the direct vision-model path",
    "Gemma4ForConditionalGeneration": "Gemma4 is not built in this framework",
    "SiglipVisionModel": "use SiglipAdapter(model).to_rpu()",
    "Qwen3_5ForConditionalGeneration": "use Qwen3_5Adapter(model).to_rpu() with Qwen3_5Cache",
    "Qwen3VLForConditionalGeneration": "use RPUModelForConditionalGeneration.from_pretrained(...)",
    "LlamaForCausalLM": "use RPUModelForCausalLM.from_pretrained(...) and .to('rpu')",
    "Qwen3ForCausalLM": "use RPUModelForCausalLM.from_pretrained(...) and .to('rpu')",
}


def resolve_loader_device(device, *, entry_point: str) -> bool:
    """True when the caller asked for the accelerator (``rpu`` / ``rpu:N`` / ``cuda``)."""
    if device is None:
        return False
    if not isinstance(device, (str, torch.device)):
        raise ValueError(f"{entry_point}: device must be None, cpu, rpu or cuda; got {device!r}")
    name = str(device).lower()
    if name.startswith("rpu") or name.startswith("cuda"):
        return True
    if name.startswith("cpu"):
        return False
    raise ValueError(f"{entry_point}: device must be None, cpu, rpu or cuda; got {device!r}")


def resolve_config_architecture(config, *, source: str, entry_point: str, supported_builtins: Collection[str]) -> str:
    from ..adapters._manifest import BUILTIN_ADAPTERS
    archs = getattr(config, "architectures", None)
    if not isinstance(archs, (list, tuple)) or not archs or any(not isinstance(a, str) or not a.strip() for a in archs):
        raise UnsupportedModelError(f"HF config at {source!r} must define `architectures` as a non-empty list of "
                                    f"non-empty strings; got {archs!r}. Cannot dispatch through {entry_point}.")
    arch = archs[0]
    if arch in {e[0] for e in BUILTIN_ADAPTERS} and arch not in supported_builtins:
        raise UnsupportedModelError(f"{entry_point} does not support built-in HF architecture {arch!r}; "
                                    f"{_ROUTES.get(arch, 'use its model-specific adapter')}.")
    return arch


def checkpoint_tensor_getter(path: str) -> Callable[[str], torch.Tensor]:
    """Lazy tensor access into a local safetensors checkpoint (single file or sharded index):
    weights stream from disk straight into the engine's packer, one tensor at a time."""
    from safetensors import safe_open
    root = Path(path)
    index = root / "model.safetensors.index.json"
    if index.is_file():
        weight_map: Dict[str, str] = json.loads(index.read_text())["weight_map"]
    else:
        single = root / "model.safetensors"
        if not single.is_file():
            raise UnsupportedModelError(f"no safetensors checkpoint under {path!r}")
        with safe_open(str(single), framework="pt") as f:
            weight_map = {k: "model.safetensors" for k in f.keys()}
    handles: Dict[str, object] = {}

    def get(name: str) -> torch.Tensor:
        if name not in weight_map:
            raise KeyError(name)
        shard = weight_map[name]
        if shard not in handles:
            handles[shard] = safe_open(str(root / shard), framework="pt")
        return handles[shard].get_tensor(name)

    get.names = frozenset(weight_map)  # type: ignore[attr-defined]
    return get


__all__ = ["resolve_loader_device", "resolve_config_architecture", "checkpoint_tensor_getter"]
