"""Check a W8A16 checkpoint against the 16-bit checkpoint it was converted from.

    python -m rhinoforge_b200.quant.verify_qwen3_w8a16 --src FP16_CKPT --quant W8A16_CKPT [--min-cosine 0.999]
        [--samples 64]

For every tensor of the source: a quantised projection must be int8 with an fp16 scale of one entry per output row,
its dequantised form must match the source (cosine >= ``--min-cosine``, every |error| <= half a quantisation step + fp16
rounding), and a random-activation product through ``(x . q^T) * scale`` must agree with the 16-bit product; every other
tensor must be unchanged up to the fp16 cast.  ``config.json`` must carry a ``quant_config`` whose flags agree with what
is found.  Exit code 0 = consistent.  Reference: ``python/rpu_backend/quant/verify_qwen3_w8a16.py``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ._checkpoint import checkpoint_layout, scale_name
from ._common import cosine, dequantize_linear_per_channel, reference_linear


def _load_all(root: Path) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    shards, _, _ = checkpoint_layout(root)
    out: Dict[str, torch.Tensor] = {}
    for s in shards:
        out.update(load_file(root / s))
    return out


def verify(src, quant, *, min_cosine: float = 0.999, samples: int = 64, seed: int = 0) -> dict:
    src, quant = Path(src).expanduser().resolve(), Path(quant).expanduser().resolve()
    a, b = _load_all(src), _load_all(quant)
    cfg = json.loads((quant / "config.json").read_text())
    qc = cfg.get("quant_config")
    problems: List[str] = []
    if not isinstance(qc, dict) or qc.get("method") != "w8a16":
        problems.append("config.json has no quant_config with method w8a16")
        qc = {}
    g = torch.Generator().manual_seed(seed)
    report = {"quantized": 0, "copied": 0, "worst_cosine": 1.0, "worst_rel_product_error": 0.0}
    for name, w in sorted(a.items()):
        if name not in b:
            problems.append(f"{name}: missing from the quantised checkpoint")
            continue
        q = b[name]
        if q.dtype == torch.int8:
            s = b.get(scale_name(name))
            if s is None or s.dtype != torch.float16 or tuple(s.shape) != (w.shape[0],):
                problems.append(f"{name}: weight_scale missing or not fp16 [out]")
                continue
            deq = dequantize_linear_per_channel(q, s).float()
            ref = w.to(torch.float16).float()
            c = cosine(deq, ref)
            step = s.float()[:, None]
            if c < min_cosine:
                problems.append(f"{name}: cosine {c:.6f} < {min_cosine}")
            if bool(((deq - ref).abs() > 0.5 * step * 1.01 + 1e-3 * ref.abs() + 1e-6).any()):
                problems.append(f"{name}: an element is off by more than half a quantisation step")
            x = torch.randn(samples, w.shape[1], generator=g)
            want, got = x @ ref.t(), reference_linear(x, q, s)
            rel = float((got - want).norm() / want.norm().clamp_min(1e-30))
            report["worst_cosine"] = min(report["worst_cosine"], c)
            report["worst_rel_product_error"] = max(report["worst_rel_product_error"], rel)
            report["quantized"] += 1
        else:
            if w.is_floating_point():
                if not torch.equal(q, w.to(torch.float16)):
                    problems.append(f"{name}: 16-bit tensor changed")
            elif not torch.equal(q, w):
                problems.append(f"{name}: tensor changed")
            report["copied"] += 1
    head_int8 = "lm_head.weight" in b and b["lm_head.weight"].dtype == torch.int8
    if qc and bool(qc.get("quantized_lm_head", False)) != head_int8:
        problems.append("quant_config.quantized_lm_head disagrees with the lm_head tensor")
    extra = sorted(n for n in b if n not in a and not n.endswith(".weight_scale") and n != "lm_head.weight")
    if extra:
        problems.append(f"unexpected tensors: {extra[:4]}")
    report["problems"] = problems
    report["ok"] = not problems
    return report


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src", required=True)
    ap.add_argument("--quant", required=True)
    ap.add_argument("--min-cosine", type=float, default=0.999)
    ap.add_argument("--samples", type=int, default=64)
    a = ap.parse_args(argv)
    try:
        rep = verify(a.src, a.quant, min_cosine=a.min_cosine, samples=a.samples)
    except (FileNotFoundError, KeyError, ValueError) as e:
        print(f"[verify_qwen3_w8a16] error: {e}", file=sys.stderr)
        return 2
    print(json.dumps({k: v for k, v in rep.items() if k != "problems"}, indent=1))
    for p in rep["problems"]:
        print(f"[verify_qwen3_w8a16] {p}", file=sys.stderr)
    return 0 if rep["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
