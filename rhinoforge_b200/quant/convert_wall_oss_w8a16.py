"""Offline W8A16 conversion of a Wall-OSS checkpoint: every 2-D floating ``*.weight`` except the skipped modules.

    python -m rhinoforge_b200.quant.convert_wall_oss_w8a16 --src CKPT --dst OUT [--skip-modules embed_tokens,...]

Per output channel, symmetric int8: a qualifying ``<name>.weight`` ``[N, K]`` becomes int8 plus ``<name>.weight_scale``
fp16 ``[N]`` - decoder expert projections, the vision transformer blocks and the action pre-processor alike (the
reference's tested ``wall-oss-0.5-w8a16`` checkpoint quantises 422 tensors this way, everything 2-D but the token
embedding).  Other tensors keep their dtype; side files are copied; the marker is the sidecar
``rpu_quant_config.json`` with the list of quantised names' count and the skip list.  Reference behaviour:
``python/rpu_backend/quant/convert_wall_oss_w8a16.py:1-60``.  (The Wall-OSS policy itself is not built in this framework;
the converter is a checkpoint tool and does not need it.)
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch

from ._checkpoint import rewrite_checkpoint, scale_name
from ._common import quantize_linear_per_channel

DEFAULT_SKIP_MODULES = ("embed_tokens",)
SIDECAR = "rpu_quant_config.json"


def wants_int8(name: str, t: torch.Tensor, skip_modules: Sequence[str]) -> bool:
    return name.endswith(".weight") and t.dim() == 2 and t.is_floating_point() and not any(s in name for s in skip_modules)


def convert_checkpoint(src, dst, *, skip_modules: Sequence[str] = DEFAULT_SKIP_MODULES) -> dict:
    skip = tuple(s for s in skip_modules if s)
    n = {"quantized": 0}

    def transform(name: str, t: torch.Tensor) -> Dict[str, torch.Tensor]:
        if not wants_int8(name, t, skip):
            return {name: t}
        q, s = quantize_linear_per_channel(t)
        n["quantized"] += 1
        return {name: q, scale_name(name): s}

    sidecar = {"source": Path(src).name, "method": "w8a16", "mode": "per_channel_symmetric", "qaxis": 0, "skip_modules": list(skip),
               "scope": "all_2d_weights"}
    stats = rewrite_checkpoint(src, dst, transform, sidecars={SIDECAR: sidecar}, drop_files=(SIDECAR,),
                               tag="convert_wall_oss_w8a16")
    stats["n_quantized"] = n["quantized"]
    return stats


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src", required=True, help="16-bit Wall-OSS checkpoint directory")
    ap.add_argument("--dst", required=True, help="output directory (must not exist)")
    ap.add_argument("--skip-modules", default=",".join(DEFAULT_SKIP_MODULES), help="comma-separated name substrings kept 16-bit")
    a = ap.parse_args(argv)
    try:
        st = convert_checkpoint(a.src, a.dst, skip_modules=[s.strip() for s in a.skip_modules.split(",")])
    except (FileExistsError, FileNotFoundError, TypeError, ValueError) as e:
        print(f"[convert_wall_oss_w8a16] error: {e}", file=sys.stderr)
        return 1
    print(f"[convert_wall_oss_w8a16] {Path(a.src).resolve()} -> {Path(a.dst).resolve()}: {st['n_quantized']} weights, "
          f"{st['bytes_in'] / 1e9:.2f} GB -> {st['bytes_out'] / 1e9:.2f} GB")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
