"""Checks that a quantised checkpoint and a 16-bit checkpoint really are a converted / source pair.

Mixed-precision Wall-OSS modes load two directories at once - the quantised projections from one, everything the mode
keeps in 16 bits from the other - and a wrong pairing (two sizes of the model, a checkpoint quantised from a different
fine-tune, the two arguments swapped) produces a model that runs and is silently wrong.  The check runs on metadata only,
before any tensor is read.  Reference behaviour: ``python/rpu_backend/adapters/wall_oss/checkpoint_validation.py:31-164``.

A pair is accepted when

* the quantised directory declares the expected method, in the ``rpu_quant_config.json`` sidecar or in
  ``config.json["quant_config"]`` (both present and disagreeing is an error);
* the 16-bit directory declares no quantisation at all;
* the quantised directory's ``source`` (a directory name, resolved against the quantised directory's parent, or an
  absolute path) exists and *is* the 16-bit directory;
* the two ``config.json`` files agree on every field except the ones a conversion legitimately changes
  (``quant_config``, ``dtype``, ``torch_dtype``).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional, Tuple, Union

from .convert_wall_oss import QUANT_SUFFIXES, SIDECAR

PathLike = Union[str, Path]
REPRESENTATION_KEYS = frozenset({"quant_config", "dtype", "torch_dtype"})
RTC_INT8_SUFFIX = "moe.experts.0.down_proj.weight"
RTC_GROUP_SIZE = 32


def _json_object(path: Path) -> dict:
    with path.open(encoding="utf-8") as f:
        body = json.load(f)
    if not isinstance(body, dict):
        raise ValueError(f"expected a JSON object in {path}")
    return body


def quant_metadata(ckpt: Path, config: dict) -> Optional[dict]:
    """The quantisation record of a checkpoint directory, or ``None`` for a plain one."""
    side = _json_object(ckpt / SIDECAR) if (ckpt / SIDECAR).is_file() else None
    inline = config.get("quant_config")
    if inline is not None and not isinstance(inline, dict):
        raise ValueError(f"expected quant_config to be an object in {ckpt / 'config.json'}")
    if side is not None and inline is not None:
        a, b = (str(m.get("method", "")).lower() for m in (side, inline))
        if a != b:
            raise ValueError(f"conflicting quantization metadata in {ckpt}: sidecar={a!r}, config={b!r}")
    return inline if side is None else side


def _resolve_source(quant_dir: Path, meta: dict, label: str) -> Path:
    src = meta.get("source")
    if not src:
        raise ValueError(f"{label} checkpoint {quant_dir} has no source provenance metadata")
    cand = Path(str(src))
    if not cand.is_absolute():
        cand = quant_dir.parent / cand
    try:
        return cand.resolve(strict=True)
    except FileNotFoundError as e:
        raise ValueError(f"{label} source provenance cannot be resolved exactly: source={src!r}, "
                         f"resolved_candidate={str(cand)!r}") from e


def validate_checkpoint_pair(quant_ckpt_dir: PathLike, fp16_ckpt_dir: PathLike, *, expected_method: str,
                             label: str) -> Tuple[dict, dict, dict]:
    """``(quantised config, 16-bit config, quantisation record)`` of an accepted pair; ``ValueError`` otherwise."""
    qdir, fdir = Path(quant_ckpt_dir), Path(fp16_ckpt_dir)
    qcfg, fcfg = _json_object(qdir / "config.json"), _json_object(fdir / "config.json")
    meta = quant_metadata(qdir, qcfg)
    method = str(meta.get("method", "")).lower() if meta is not None else ""
    if method != expected_method:
        raise ValueError(f"quantized ckpt_dir must be a {label} checkpoint with method={expected_method!r}; got "
                         f"{method or 'unquantized'} at {qdir}")
    plain = quant_metadata(fdir, fcfg)
    if plain is not None:
        raise ValueError(f"fp16_ckpt_dir must be an unquantized source checkpoint; found method={plain.get('method')!r} "
                         f"at {fdir}")
    declared, given = _resolve_source(qdir, meta, label), fdir.resolve(strict=True)
    if declared != given:
        raise ValueError(f"{label} and FP16 checkpoints are not a declared source pair: quantized source="
                         f"{str(declared)!r}, fp16_ckpt_dir={str(given)!r}")
    differing = sorted(k for k in (set(qcfg) | set(fcfg)) - REPRESENTATION_KEYS if qcfg.get(k) != fcfg.get(k))
    if differing:
        raise ValueError(f"{label} and FP16 checkpoints are not architecture-compatible; mismatched config fields: "
                         f"{differing}")
    return qcfg, fcfg, meta


def validate_w8_nvfp4_checkpoint_pair(w8_ckpt_dir: PathLike, fp16_ckpt_dir: PathLike) -> Tuple[dict, dict]:
    """The W8A16 + 16-bit pair of the mode that keeps W8 projections and re-quantises the rest to NVFP4 at load."""
    q, f, _ = validate_checkpoint_pair(w8_ckpt_dir, fp16_ckpt_dir, expected_method="w8a16", label="W8A16")
    return q, f


def validate_rtc_w4_checkpoint_pair(w4_ckpt_dir: PathLike, fp16_ckpt_dir: PathLike) -> Tuple[dict, dict]:
    """The real-time-chunking composition: group-32 INT4 for seven expert projections, expert 0's down projection kept
    INT8, everything else from the 16-bit source."""
    q, f, meta = validate_checkpoint_pair(w4_ckpt_dir, fp16_ckpt_dir, expected_method="w4a16", label="RTC W4A16")
    int4_expected = [s for s in QUANT_SUFFIXES if s != RTC_INT8_SUFFIX]
    exact = (meta.get("mode") in ("group_wise_symmetric", "per_group_symmetric")
             and meta.get("group_size") == RTC_GROUP_SIZE
             and meta.get("int8_suffixes") == [RTC_INT8_SUFFIX]
             and meta.get("int4_suffixes") == int4_expected)
    if not exact:
        raise ValueError("Wall-OSS RTC W4A16 requires the exact seven group-wise INT4 projection suffixes with "
                         f"group_size={RTC_GROUP_SIZE} and expert-0 down_proj retained as INT8")
    return q, f


__all__ = ["validate_checkpoint_pair", "validate_w8_nvfp4_checkpoint_pair", "validate_rtc_w4_checkpoint_pair",
           "quant_metadata", "REPRESENTATION_KEYS"]
