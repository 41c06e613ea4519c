"""Shard-by-shard rewriting of a safetensors checkpoint directory (shared by the offline converters).

``rewrite_checkpoint(src, dst, transform)`` walks ``model.safetensors`` or the shards of
``model.safetensors.index.json``, hands every tensor to ``transform(name, tensor) -> {new_name: tensor}``, keeps the
weight map in step with added names, copies the side files, lets the caller patch ``config.json`` / add sidecars, and
publishes the result atomically (temporary directory renamed at the end; an existing ``dst`` is never overwritten).
"""
from __future__ import annotations

import json
import os
import shutil
from pathlib import Path
from typing import Callable, Dict, Iterable, Optional

import torch

Transform = Callable[[str, torch.Tensor], Dict[str, torch.Tensor]]


def checkpoint_layout(src: Path):
    idx = src / "model.safetensors.index.json"
    if idx.is_file():
        index = json.loads(idx.read_text())
        wm = dict(index["weight_map"])
        return sorted(set(wm.values())), wm, index
    if (src / "model.safetensors").is_file():
        return ["model.safetensors"], None, None
    raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json in {src}")


def tensor_bytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def rewrite_checkpoint(src, dst, transform: Transform, *, config_patch: Optional[Callable[[dict], dict]] = None,
                       sidecars: Optional[Dict[str, dict]] = None, drop_files: Iterable[str] = (),
                       tag: str = "convert") -> dict:
    from safetensors.torch import load_file, save_file
    src, dst = Path(src).expanduser().resolve(), Path(dst).expanduser().resolve()
    if not src.is_dir():
        raise FileNotFoundError(f"--src is not a directory: {src}")
    if dst.exists():
        raise FileExistsError(f"--dst already exists, refusing to overwrite: {dst}")
    shards, weight_map, index = checkpoint_layout(src)
    tmp = dst.with_name(f".{dst.name}.tmp-{os.getpid()}")
    if tmp.exists():
        raise FileExistsError(f"temporary output already exists: {tmp}")
    stats = {"n_shards": len(shards), "n_tensors_in": 0, "n_tensors_out": 0, "bytes_in": 0, "bytes_out": 0}
    new_map = {} if weight_map is not None else None
    try:
        tmp.mkdir(parents=True)
        for i, shard in enumerate(shards, 1):
            print(f"[{tag}] shard {i}/{len(shards)}: {shard}", flush=True)
            tensors = load_file(src / shard)
            out: Dict[str, torch.Tensor] = {}
            for name in sorted(tensors):
                t = tensors[name]
                stats["n_tensors_in"] += 1
                stats["bytes_in"] += tensor_bytes(t)
                for new_name, nt in transform(name, t).items():
                    out[new_name] = nt.contiguous()
                    stats["n_tensors_out"] += 1
                    stats["bytes_out"] += tensor_bytes(nt)
                    if new_map is not None:
                        new_map[new_name] = shard
            save_file(out, tmp / shard, metadata={"format": "pt"})
            del tensors, out
        if index is not None:
            index = dict(index)
            index["metadata"] = {**index.get("metadata", {}), "total_size": stats["bytes_out"]}
            index["weight_map"] = dict(sorted(new_map.items()))
            (tmp / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))
        cfg_path = src / "config.json"
        if cfg_path.is_file():
            config = json.loads(cfg_path.read_text())
            if config_patch is not None:
                config = config_patch(config)
            (tmp / "config.json").write_text(json.dumps(config, indent=2))
        for name, body in (sidecars or {}).items():
            (tmp / name).write_text(json.dumps(body, indent=2))
        skip = set(shards) | {"model.safetensors", "model.safetensors.index.json", "config.json"} | set(drop_files) \
            | set(sidecars or {})
        for p in sorted(src.iterdir()):
            if p.is_file() and p.name not in skip:
                shutil.copy2(p, tmp / p.name)
        tmp.rename(dst)
    except Exception:
        shutil.rmtree(tmp, ignore_errors=True)
        raise
    return stats


def scale_name(weight_name: str) -> str:
    return weight_name[:-len(".weight")] + ".weight_scale"


__all__ = ["rewrite_checkpoint", "checkpoint_layout", "scale_name", "tensor_bytes"]
