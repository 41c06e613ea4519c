"""Offline W4A16 conversion of a Qwen3 checkpoint: packed 4-bit projections with group-wise scales.

    python -m rhinoforge_b200.quant.convert_qwen3_w4a16 --src CKPT --dst OUT [--group-size 32|64|128]
        [--skip-modules NAME ...]

Each decoder projection ``<name>.weight`` ``[out, in]`` becomes ``<name>.weight`` uint8 ``[out, in/2]`` (two signed
4-bit values per byte, low nibble first) plus ``<name>.weight_scale`` fp16 ``[out, in/group]``; other tensors are stored
as fp16.  ``config.json`` gains ``quant_config = {method: "w4a16", mode: "per_group_symmetric", group_size, qaxis: 0,
skip_modules}``.  The packed layout is the one of ``quant/int4_pgrp_pack.py``; the loader dequantises it to the 16-bit
GEMM path (``quant.int4_pgrp_pack.dequantize_int4_pgrp``) - a 4-bit device GEMM is not part of this build.
Reference behaviour: ``python/rpu_backend/quant/convert_qwen3_w4a16.py``.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ._checkpoint import rewrite_checkpoint, scale_name
from .convert_qwen3 import PROJECTION_SUFFIXES
from .int4_pgrp_pack import GROUP_SIZES, quantize_pack_int4_pgrp


def convert_checkpoint(src, dst, *, group_size: int = 32, skip_modules: Optional[List[str]] = None) -> dict:
    if group_size not in GROUP_SIZES:
        raise ValueError(f"--group-size must be one of {GROUP_SIZES}")
    skip = list(skip_modules or [])
    n = {"quantized": 0}

    def transform(name: str, t: torch.Tensor) -> Dict[str, torch.Tensor]:
        if name.endswith(PROJECTION_SUFFIXES) and not any(s in name for s in skip) and t.is_floating_point():
            if t.shape[1] % group_size:
                raise ValueError(f"{name}: in_features {t.shape[1]} is not a multiple of the group size {group_size}")
            packed, scale = quantize_pack_int4_pgrp(t, group_size)
            n["quantized"] += 1
            return {name: packed, scale_name(name): scale}
        return {name: t.to(torch.float16) if t.is_floating_point() else t}

    def patch(config: dict) -> dict:
        config["torch_dtype"] = config["dtype"] = "float16"
        config["quant_config"] = {"method": "w4a16", "mode": "per_group_symmetric", "group_size": group_size, "qaxis": 0,
                                  "packing": "int4x2_low_nibble_first", "skip_modules": skip}
        return config

    stats = rewrite_checkpoint(src, dst, transform, config_patch=patch, tag="convert_qwen3_w4a16")
    stats["n_quantized"] = n["quantized"]
    return stats


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--group-size", type=int, default=32, choices=GROUP_SIZES)
    ap.add_argument("--skip-modules", nargs="*", default=[])
    a = ap.parse_args(argv)
    try:
        st = convert_checkpoint(a.src, a.dst, group_size=a.group_size, skip_modules=a.skip_modules)
    except (FileExistsError, FileNotFoundError, TypeError, ValueError) as e:
        print(f"[convert_qwen3_w4a16] error: {e}", file=sys.stderr)
        return 1
    print(f"[convert_qwen3_w4a16] {Path(a.src).resolve()} -> {Path(a.dst).resolve()}: {st['n_quantized']} projections, "
          f"{st['bytes_in'] / 1e9:.2f} GB -> {st['bytes_out'] / 1e9:.2f} GB")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
