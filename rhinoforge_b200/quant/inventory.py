"""Header-only inventory check of a W8A16 checkpoint: what is int8, what has a scale, what is left in 16 bits.

A W8A16 checkpoint that is *almost* right - one projection left in bf16, a scale of the wrong length, a tensor listed in
the index but absent from its shard - loads and then computes garbage or fails half-way through a 30 GB transfer.  The
safetensors header carries every tensor's name, dtype and shape, so all of this can be decided before a single weight is
read.  The reference performs the same checks while building its load plan for the Qwen3-VL-32B W8A16 profile, against a
meta-device model (``python/rpu_backend/quant/load.py:360-512``); here the expected inventory follows from the tensor
names alone, because loading is streamed through a getter and no host-side module tree exists.

Rules, for tensors under a decoder layer (``...layers.<i>.``) whose name ends in a quantised projection suffix:

* the weight is ``I8`` and 2-D, and ``<name>_scale`` exists, is ``F16`` and has one entry per output row;
* with ``require_all=True`` (default) a projection left in a floating dtype is an error, otherwise it is listed under
  ``unquantized``;
* a ``*.weight_scale`` without its int8 weight is an error; every other tensor must be floating (or integer buffers
  named in ``allow_integer``);
* a tensor name may appear in one shard only; with an index file, its weight map must name exactly the tensors found,
  each in the shard that holds it.
"""
from __future__ import annotations

import json
import re
from pathlib import Path
from typing import Any, Dict, Iterable, List, Sequence, Tuple

from .convert_qwen3 import QUANT_PROJ_SUFFIXES, scale_name
from .load import _shards

FLOAT_DTYPES = frozenset({"F64", "F32", "F16", "BF16"})
ELEMENT_BYTES = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I8": 1, "U8": 1, "I32": 4, "I64": 8, "BOOL": 1, "I16": 2}
_LAYER = re.compile(r"(?:^|\.)layers\.(\d+)\.")
_VISION = re.compile(r"(?:^|\.)(visual|vision_tower|vision_model)\.")


def _headers(shards: Sequence[Path]) -> Dict[str, Tuple[str, Tuple[int, ...], str]]:
    """``{tensor name: (dtype, shape, shard file name)}`` from the headers of ``shards``."""
    from safetensors import safe_open
    seen: Dict[str, Tuple[str, Tuple[int, ...], str]] = {}
    for shard in shards:
        with safe_open(str(shard), framework="pt") as f:
            for name in f.keys():
                if name in seen:
                    raise KeyError(f"W8A16 checkpoint tensor {name!r} appears more than once ({seen[name][2]}, {shard.name})")
                sl = f.get_slice(name)
                seen[name] = (str(sl.get_dtype()), tuple(int(d) for d in sl.get_shape()), shard.name)
    return seen


def is_decoder_projection(name: str, suffixes: Sequence[str] = QUANT_PROJ_SUFFIXES) -> bool:
    """A language-model decoder projection: under ``layers.<i>.``, not in a vision tower, with a quantised suffix."""
    return bool(_LAYER.search(name)) and not _VISION.search(name) and name.endswith(tuple(suffixes))


def inspect_w8a16_checkpoint(ckpt_dir, *, suffixes: Sequence[str] = QUANT_PROJ_SUFFIXES, require_all: bool = True,
                             extra_int8: Iterable[str] = (), allow_integer: Iterable[str] = ()) -> Dict[str, Any]:
    """Validate the inventory (rules in the module docstring) and return the load plan::

        {"tensor_shards": {name: shard}, "int8": [...], "scales": [...], "unquantized": [...],
         "layers": [[names of layer 0], ...], "nondecoder": [...], "bytes": total}

    ``extra_int8`` names tensors outside the decoder layers that are quantised as well (an untied ``lm_head.weight``).
    Raises ``FileNotFoundError`` / ``KeyError`` / ``TypeError`` / ``ValueError`` with the offending tensor names."""
    root = Path(ckpt_dir)
    meta = _headers(_shards(root))
    extra = set(extra_int8)
    integer_ok = set(allow_integer)
    int8: List[str] = []
    scales: List[str] = []
    loose: List[str] = []
    for name, (dtype, shape, _) in meta.items():
        if name.endswith(".weight_scale"):
            owner = name[:-len("_scale")]
            if owner not in meta or meta[owner][0] != "I8":
                raise KeyError(f"W8A16 checkpoint has unexpected scale {name!r} (no int8 tensor {owner!r})")
            if dtype != "F16":
                raise TypeError(f"W8A16 scale {name!r} must be fp16, got {dtype}")
            if shape != (meta[owner][1][0],):
                raise ValueError(f"W8A16 scale {name!r} has shape {shape}, expected {(meta[owner][1][0],)}")
            scales.append(name)
        elif is_decoder_projection(name, suffixes) or name in extra:
            if dtype == "I8":
                if len(shape) != 2:
                    raise ValueError(f"W8A16 projection {name!r} must be 2-D, got shape {shape}")
                if scale_name(name) not in meta:
                    raise KeyError(f"W8A16 projection {name!r} has no {scale_name(name)!r}")
                int8.append(name)
            elif dtype in FLOAT_DTYPES and not require_all:
                loose.append(name)
            else:
                raise TypeError(f"W8A16 projection {name!r} must be int8, got {dtype}")
        elif dtype == "I8":
            raise TypeError(f"W8A16 checkpoint quantises {name!r}, which is not a decoder projection")
        elif dtype not in FLOAT_DTYPES and name not in integer_ok:
            raise TypeError(f"W8A16 non-projection tensor {name!r} must be floating, got {dtype}")

    index = root / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map")
        if not isinstance(weight_map, dict):
            raise KeyError("W8A16 checkpoint index has no object-valued weight_map")
        if set(weight_map) != set(meta):
            raise KeyError(f"W8A16 checkpoint index and shards disagree: only in shards {sorted(set(meta) - set(weight_map))[:8]}, "
                           f"only in index {sorted(set(weight_map) - set(meta))[:8]}")
        moved = sorted(n for n, s in weight_map.items() if meta[n][2] != s)
        if moved:
            raise KeyError(f"W8A16 checkpoint index points to the wrong shard for {moved[:8]}")

    depth = 1 + max((int(m.group(1)) for m in map(_LAYER.search, meta) if m and not _VISION.search(m.string)), default=-1)
    layers: List[List[str]] = [[] for _ in range(depth)]
    nondecoder: List[str] = []
    for name in sorted(meta):
        m = _LAYER.search(name)
        (layers[int(m.group(1))] if m and not _VISION.search(name) else nondecoder).append(name)
    per_layer = {len([n for n in names if n in set(int8)]) for names in layers}
    if len(per_layer) > 1:
        raise KeyError(f"W8A16 decoder layers hold different numbers of int8 projections: {sorted(per_layer)}")
    total = 0
    for dtype, shape, _ in meta.values():
        count = ELEMENT_BYTES.get(dtype, 0)
        for d in shape:
            count *= d
        total += count
    return {"tensor_shards": {n: v[2] for n, v in meta.items()}, "int8": sorted(int8), "scales": sorted(scales),
            "unquantized": sorted(loose), "layers": layers, "nondecoder": nondecoder, "bytes": total}


__all__ = ["inspect_w8a16_checkpoint", "is_decoder_projection", "FLOAT_DTYPES"]
