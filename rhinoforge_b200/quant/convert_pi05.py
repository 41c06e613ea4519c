"""Offline W8A16 (or 4-bit probe) conversion of a Pi0.5 checkpoint.

    python -m rhinoforge_b200.quant.convert_pi05 --src CKPT --dst OUT [--bits 8|4] [--targets vlm expert]
        [--keep-int8-suffixes SUFFIX ...]

Quantised: the seven projections of every Gemma layer of the prefix backbone (``...paligemma.model.language_model.
layers.*``) and of the action expert (``...gemma_expert.model.layers.*``), per output channel, symmetric.  Left as they
are: SigLIP, the adaRMS conditioning denses, the action / time projections, embeddings, norms.  ``--bits 4`` stores
values of [-8, 7] in int8 containers - the W8A16 kernels run them unchanged, so it is a numerical probe of 4-bit
weights, not a size reduction; ``--keep-int8-suffixes`` exempts projections from it.  The result carries the sidecar
``rpu_quant_config.json`` (not a ``config.json`` edit: the policy config is a LeRobot file) and deliberately no
``model_remapped.safetensors``: the loader's remap cache is rebuilt from the quantised tensors.
Reference behaviour: ``python/rpu_backend/quant/convert_pi05.py:1-60,207-310``.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch

from ._checkpoint import rewrite_checkpoint, scale_name
from ._common import quantize_linear_per_channel

EXPERT_ANCHOR = "paligemma_with_expert.gemma_expert.model.layers."
VLM_ANCHOR = "paligemma_with_expert.paligemma.model.language_model.layers."
PROJ_SUFFIXES = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                 "self_attn.o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")
SIDECAR = "rpu_quant_config.json"


def target_of(name: str) -> Optional[str]:
    """``"vlm"`` / ``"expert"`` for a projection this converter handles, else None."""
    if not name.endswith(PROJ_SUFFIXES):
        return None
    if EXPERT_ANCHOR in name:
        return "expert"
    if VLM_ANCHOR in name:
        return "vlm"
    return None


def bits_for(name: str, bits: int, keep_int8: Sequence[str]) -> int:
    return 8 if bits == 4 and any(name.endswith(s) for s in keep_int8) else bits


def convert_checkpoint(src, dst, *, bits: int = 8, targets: Sequence[str] = ("vlm", "expert"),
                       keep_int8_suffixes: Sequence[str] = ()) -> dict:
    if bits not in (4, 8):
        raise ValueError("--bits must be 4 or 8")
    bad = [t for t in targets if t not in ("vlm", "expert")]
    if bad:
        raise ValueError(f"unknown targets {bad}")
    keep = tuple(s if s.endswith(".weight") else s + ".weight" for s in keep_int8_suffixes)
    counts: Dict[str, int] = {"vlm": 0, "expert": 0, "int8": 0, "int4": 0}

    def transform(name: str, t: torch.Tensor) -> Dict[str, torch.Tensor]:
        tgt = target_of(name)
        if tgt is None or tgt not in targets or t.dtype == torch.int8:
            return {name: t}
        if not t.is_floating_point():
            raise TypeError(f"cannot quantize non-floating tensor {name!r} ({t.dtype})")
        b = bits_for(name, bits, keep)
        q, s = quantize_linear_per_channel(t, bits=b)
        counts[tgt] += 1
        counts["int8" if b == 8 else "int4"] += 1
        return {name: q, scale_name(name): s}

    sidecar = {"method": "w8a16" if bits == 8 else "w4a16_probe_in_int8", "mode": "per_channel_symmetric", "qaxis": 0,
               "bits": bits, "targets": list(targets), "keep_int8_suffixes": list(keep),
               "quantized_suffixes": list(PROJ_SUFFIXES)}
    stats = rewrite_checkpoint(src, dst, transform, sidecars={SIDECAR: sidecar},
                               drop_files=("model_remapped.safetensors", SIDECAR), tag="convert_pi05")
    stats.update(counts)
    return stats


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src", required=True, help="source Pi0.5 checkpoint directory")
    ap.add_argument("--dst", required=True, help="output directory (must not exist)")
    ap.add_argument("--bits", type=int, default=8, choices=(4, 8))
    ap.add_argument("--targets", nargs="+", default=["vlm", "expert"], choices=("vlm", "expert"))
    ap.add_argument("--keep-int8-suffixes", nargs="*", default=[],
                    help="projection suffixes kept at 8 bits under --bits 4 (e.g. self_attn.o_proj)")
    a = ap.parse_args(argv)
    try:
        st = convert_checkpoint(a.src, a.dst, bits=a.bits, targets=a.targets, keep_int8_suffixes=a.keep_int8_suffixes)
    except (FileExistsError, FileNotFoundError, TypeError, ValueError) as e:
        print(f"[convert_pi05] error: {e}", file=sys.stderr)
        return 1
    print(f"[convert_pi05] {Path(a.src).resolve()} -> {Path(a.dst).resolve()}: vlm {st['vlm']} expert {st['expert']} "
          f"projections ({st['int8']} int8, {st['int4']} 4-bit), {st['bytes_in'] / 1e9:.2f} GB -> {st['bytes_out'] / 1e9:.2f} GB")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
