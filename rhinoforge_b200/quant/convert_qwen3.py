"""Offline W8A16 conversion of a Qwen3 (or Llama) Hugging Face checkpoint.

    python -m rhinoforge_b200.quant.convert_qwen3 --src CKPT --dst OUT [--quant-lm-head]
        [--quant-embed-tokens] [--skip-modules NAME ...]

The seven decoder projections (q/k/v/o/gate/up/down) become int8 with one fp16 scale per output
channel, stored as ``<name>.weight`` (int8) and ``<name>.weight_scale`` (fp16 ``[out]``) in the
same shard; every other floating tensor is stored as fp16.  ``config.json`` gains
``quant_config = {method: "w8a16", mode: "per_channel_symmetric", qaxis: 0, skip_modules,
quantized_lm_head, quantized_embed_tokens, lm_head_untied, embed_tokens_untied}``.  The output
directory is written under a temporary name and renamed at the end; an existing ``--dst`` is
never overwritten.  Checkpoint layout of the reference:
``python/rpu_backend/quant/convert_qwen3.py:25-36,112-235``.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ._common import quantize_linear_per_channel

PROJECTION_SUFFIXES = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "gate_proj.weight",
                       "up_proj.weight", "down_proj.weight")
QUANT_PROJ_SUFFIXES = PROJECTION_SUFFIXES
LM_HEAD = "lm_head.weight"
EMBED = "model.embed_tokens.weight"


def scale_name(weight_name: str) -> str:
    return weight_name[:-len(".weight")] + ".weight_scale"


@dataclass
class ConversionStats:
    n_shards: int = 0
    n_quantized: int = 0
    n_copied: int = 0
    bytes_in: int = 0
    bytes_out: int = 0

    def as_dict(self) -> dict:
        return dict(self.__dict__)


@dataclass
class _Plan:
    """What to do with each tensor name; built once, applied shard by shard."""
    skip_modules: List[str]
    quant_lm_head: bool
    quant_embed: bool
    names: set = field(default_factory=set)

    def wants_int8(self, name: str) -> bool:
        if name == LM_HEAD:
            return self.quant_lm_head
        if name == EMBED:
            return self.quant_embed
        return name.endswith(PROJECTION_SUFFIXES) and not any(s in name for s in self.skip_modules)

    @property
    def synthesize_lm_head(self) -> bool:
        return self.quant_lm_head and LM_HEAD not in self.names


def _layout(src: Path):
    idx = src / "model.safetensors.index.json"
    if idx.is_file():
        index = json.loads(idx.read_text())
        wm = dict(index["weight_map"])
        return sorted(set(wm.values())), wm, index
    if (src / "model.safetensors").is_file():
        return ["model.safetensors"], None, None
    raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json in {src}")


def _bytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def _convert_shard(tensors: Dict[str, torch.Tensor], plan: _Plan, stats: ConversionStats,
                   new_map: Optional[Dict[str, str]], shard: str) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(tensors):
        t = tensors[name]
        stats.bytes_in += _bytes(t)
        if plan.wants_int8(name) and t.dtype != torch.int8:
            if not t.is_floating_point():
                raise TypeError(f"cannot W8A16-quantize non-floating tensor {name!r} with dtype {t.dtype}")
            q, s = quantize_linear_per_channel(t)
            out[name], out[scale_name(name)] = q, s
            stats.n_quantized += 1
            stats.bytes_out += _bytes(q) + _bytes(s)
            if new_map is not None:
                new_map[scale_name(name)] = shard
        else:  # already int8 (re-conversion), a scale, a norm, an embedding ...
            keep = t.to(torch.float16) if t.is_floating_point() else t
            out[name] = keep
            stats.n_copied += 1
            stats.bytes_out += _bytes(keep)
        if name == EMBED and plan.synthesize_lm_head:
            # tied checkpoint: derive an untied int8 lm_head from the embedding rows
            if plan.quant_embed:
                q, s = out[EMBED].clone(), out[scale_name(EMBED)].clone()
            else:
                q, s = quantize_linear_per_channel(t)
            out[LM_HEAD], out[scale_name(LM_HEAD)] = q, s
            stats.n_quantized += 1
            stats.bytes_out += _bytes(q) + _bytes(s)
            if new_map is not None:
                new_map[LM_HEAD] = shard
                new_map[scale_name(LM_HEAD)] = shard
    return out


def convert_checkpoint(src, dst, skip_modules: List[str], *, quant_lm_head: bool = False,
                       quant_embed_tokens: bool = False) -> dict:
    from safetensors.torch import load_file, save_file
    src, dst = Path(src).expanduser().resolve(), Path(dst).expanduser().resolve()
    if not src.is_dir():
        raise FileNotFoundError(f"--src is not a directory: {src}")
    if dst.exists():
        raise FileExistsError(f"--dst already exists, refusing to overwrite: {dst}")
    shards, weight_map, index = _layout(src)
    tmp = dst.with_name(f".{dst.name}.tmp-{os.getpid()}")
    if tmp.exists():
        raise FileExistsError(f"temporary output already exists: {tmp}")
    plan = _Plan(list(skip_modules), quant_lm_head, quant_embed_tokens)
    if weight_map is not None:
        plan.names = set(weight_map)
    stats = ConversionStats(n_shards=len(shards))
    new_map = dict(weight_map) if weight_map is not None else None
    try:
        tmp.mkdir(parents=True)
        for i, shard in enumerate(shards, 1):
            print(f"[convert_qwen3] shard {i}/{len(shards)}: {shard}", flush=True)
            tensors = load_file(src / shard)
            if weight_map is None:
                plan.names = set(tensors)
            save_file(_convert_shard(tensors, plan, stats, new_map, shard), tmp / shard, metadata={"format": "pt"})
            del tensors
        if index is not None:
            index = dict(index)
            index["metadata"] = {**index.get("metadata", {}), "total_size": stats.bytes_out}
            index["weight_map"] = dict(sorted(new_map.items()))
            (tmp / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))
        config = json.loads((src / "config.json").read_text())
        config["torch_dtype"] = config["dtype"] = "float16"
        if quant_lm_head or quant_embed_tokens:
            config["tie_word_embeddings"] = False
        config["quant_config"] = {
            "method": "w8a16", "mode": "per_channel_symmetric", "qaxis": 0,
            "skip_modules": [m for m in skip_modules if not (quant_lm_head and m == "lm_head")],
            "quantized_lm_head": bool(quant_lm_head), "quantized_embed_tokens": bool(quant_embed_tokens),
            "lm_head_untied": bool(quant_lm_head), "embed_tokens_untied": bool(quant_embed_tokens),
        }
        (tmp / "config.json").write_text(json.dumps(config, indent=2))
        skip = set(shards) | {"model.safetensors", "model.safetensors.index.json", "config.json"}
        for p in sorted(src.iterdir()):
            if p.is_file() and p.name not in skip:
                shutil.copy2(p, tmp / p.name)
        tmp.rename(dst)
    except Exception:
        shutil.rmtree(tmp, ignore_errors=True)
        raise
    return stats.as_dict()


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--skip-modules", nargs="+", default=["lm_head"], help="module-name substrings never quantised")
    ap.add_argument("--quant-lm-head", action="store_true",
                    help="int8 lm_head; derived from the embeddings (untied) when the checkpoint is tied")
    ap.add_argument("--quant-embed-tokens", action="store_true", help="int8 embeddings (needs --quant-lm-head)")
    a = ap.parse_args(argv)
    if a.quant_embed_tokens and not a.quant_lm_head:
        print("[convert_qwen3] error: --quant-embed-tokens requires --quant-lm-head", file=sys.stderr)
        return 1
    try:
        st = convert_checkpoint(a.src, a.dst, a.skip_modules, quant_lm_head=a.quant_lm_head,
                                quant_embed_tokens=a.quant_embed_tokens)
    except (FileExistsError, FileNotFoundError, TypeError, ValueError) as e:
        print(f"[convert_qwen3] error: {e}", file=sys.stderr)
        return 1
    print(f"[convert_qwen3] {Path(a.src).resolve()} -> {Path(a.dst).resolve()}")
    print(f"  shards {st['n_shards']}  quantized {st['n_quantized']}  copied {st['n_copied']}  "
          f"{st['bytes_in'] / 1e9:.2f} GB -> {st['bytes_out'] / 1e9:.2f} GB")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
