"""Offline W4A16 conversion of the Wall-OSS decoder expert projections.

    python -m rhinoforge_b200.quant.convert_wall_oss --src CKPT --dst OUT [--keep-int8 SUFFIX,...] [--group-size 0|32|64|128]

Quantised: the fused per-expert projections of both experts of every decoder layer - ``self_attn.qkv_proj_experts.{0,1}``,
``self_attn.o_proj_experts.{0,1}``, ``moe.experts.{0,1}.gate_up_proj``, ``moe.experts.{0,1}.down_proj``.  With
``--group-size 0`` (default) values of [-8, 7] are stored in int8 containers with one fp16 scale per output channel;
with a group size the weight is packed two values per byte with one scale per (channel, group) - the layouts of
``quant/_common.py`` and ``quant/int4_pgrp_pack.py``.  ``--keep-int8`` retreats listed suffixes to 8 bits.  Vision,
merger, embeddings, norms, biases and the action pre-processor are copied unchanged.  An intermediate size that the
consumer has to pad (the reference pads expert 0's 11008 to 11264 at load) is left as it is on disk.  The marker is the
sidecar ``rpu_quant_config.json``.  Reference behaviour: ``python/rpu_backend/quant/convert_wall_oss.py:1-60``.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch

from ._checkpoint import rewrite_checkpoint, scale_name
from ._common import quantize_linear_per_channel
from .int4_pgrp_pack import GROUP_SIZES, quantize_pack_int4_pgrp

QUANT_SUFFIXES = tuple(f"{stem}.{e}{tail}.weight" for stem, tail in (("self_attn.qkv_proj_experts", ""),
                                                                      ("self_attn.o_proj_experts", ""))
                       for e in (0, 1)) + tuple(f"moe.experts.{e}.{p}.weight" for p in ("gate_up_proj", "down_proj")
                                                for e in (0, 1))
SIDECAR = "rpu_quant_config.json"


def bits_for(name: str, keep_int8: Sequence[str]) -> int:
    return 8 if any(name.endswith(s) for s in keep_int8) else 4


def convert_checkpoint(src, dst, *, keep_int8: Sequence[str] = (), group_size: int = 0) -> dict:
    if group_size not in (0, *GROUP_SIZES):
        raise ValueError(f"--group-size must be 0 or one of {GROUP_SIZES}")
    keep = tuple(s if s.endswith(".weight") else s + ".weight" for s in keep_int8 if s)
    n = {"int4": 0, "int8": 0}

    def transform(name: str, t: torch.Tensor) -> Dict[str, torch.Tensor]:
        if not name.endswith(QUANT_SUFFIXES) or not t.is_floating_point() or t.dim() != 2:
            return {name: t}
        b = bits_for(name, keep)
        if b == 4 and group_size:
            if t.shape[1] % group_size:
                raise ValueError(f"{name}: in_features {t.shape[1]} is not a multiple of the group size {group_size}")
            q, s = quantize_pack_int4_pgrp(t, group_size)
        else:
            q, s = quantize_linear_per_channel(t, bits=b)
        n["int4" if b == 4 else "int8"] += 1
        return {name: q, scale_name(name): s}

    # "source" is the directory name only: converted checkpoints sit beside their source, and a build host's path must
    # not leak into the artifact; checkpoint_pair.validate_* resolves it relative to the converted directory's parent
    sidecar = {"source": Path(src).name, "method": "w4a16", "mode": "per_group_symmetric" if group_size else "per_channel_symmetric", "qaxis": 0,
               "group_size": group_size, "container": "uint8x2" if group_size else "int8",
               "int4_suffixes": [s for s in QUANT_SUFFIXES if s not in keep], "int8_suffixes": list(keep)}
    stats = rewrite_checkpoint(src, dst, transform, sidecars={SIDECAR: sidecar}, drop_files=(SIDECAR,),
                               tag="convert_wall_oss")
    stats.update(n)
    return stats


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src", required=True, help="16-bit Wall-OSS checkpoint directory")
    ap.add_argument("--dst", required=True, help="output directory (must not exist)")
    ap.add_argument("--keep-int8", default="", help="comma-separated projection suffixes kept at 8 bits")
    ap.add_argument("--group-size", type=int, default=0, help="0: one scale per output channel; 32/64/128: packed groups")
    a = ap.parse_args(argv)
    try:
        st = convert_checkpoint(a.src, a.dst, keep_int8=[s.strip() for s in a.keep_int8.split(",")], group_size=a.group_size)
    except (FileExistsError, FileNotFoundError, TypeError, ValueError) as e:
        print(f"[convert_wall_oss] error: {e}", file=sys.stderr)
        return 1
    print(f"[convert_wall_oss] {Path(a.src).resolve()} -> {Path(a.dst).resolve()}: {st['int4']} 4-bit, {st['int8']} 8-bit "
          f"projections, {st['bytes_in'] / 1e9:.2f} GB -> {st['bytes_out'] / 1e9:.2f} GB")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
