#!/usr/bin/env python3
"""RhinoVLA policy (Qwen3-VL backbone + adaRMS action expert).

This entry point validates its configuration; the model family itself is not part of this build yet, so a
real run stops with UnsupportedModelError before any checkpoint is read."""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _config import check_execution, load_toml, ok, parse_args, require_model, require_request

FAMILY = "RhinoVLA (Qwen3-VL backbone + adaRMS / QK-norm / M-RoPE action expert)"


def load_config(path) -> dict:
    config = load_toml(path)
    require_model(config)
    model = config["model"]
    for key, kind in (("dataset_key", str), ("camera_names", list), ("action_horizon", int), ("num_steps", int), ("max_seq_len", int)):
        if key in model and (not isinstance(model[key], kind) or isinstance(model[key], bool)):
            raise ValueError(f"[model].{key} must be of type {kind.__name__}")
    req = require_request(config, fields=(("instruction", str), ("noise_seed", int)))
    if not isinstance(req.get("images"), list) or not all(isinstance(p, str) for p in req["images"]):
        raise ValueError("[request].images must be a list of path strings")
    if not isinstance(req.get("instruction"), str):
        raise ValueError("[request].instruction must be a string")
    check_execution(config, {"prefill", "vision", "action"})
    return config


def main() -> int:
    args = parse_args("rhinovla.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    from rpu_backend.api.errors import UnsupportedModelError
    raise UnsupportedModelError(f"{FAMILY} is not built in this release; supported policies: Pi0.5 (examples/pi05.py)")


if __name__ == "__main__":
    raise SystemExit(main())
