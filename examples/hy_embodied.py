#!/usr/bin/env python3
"""HY-Embodied vision-language-action policy (HunYuan-VL mixture-of-transformers + action expert).

The checkpoint directory must hold model.safetensors and the tokenizer files; physical poses additionally need the
normalisation statistics ([model].norm_stats_path, JSON) and the current end-effector pose ([request].ee_pose)."""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _config import check_execution, load_toml, ok, parse_args, require_model, require_request

FAMILY = "HY-Embodied (HunYuan-VL MoT prefill + action expert)"


def load_config(path) -> dict:
    config = load_toml(path)
    require_model(config)
    model = config["model"]
    for key, kind in (("dtype", str), ("prefix_len", int), ("n_cameras", int), ("norm_stats_path", str)):
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
    args = parse_args("hy_embodied.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    from _config import load_image, resolve_checkpoint
    from rpu_backend.api import HyEmbodiedPolicy
    model, req = config["model"], config["request"]
    images = [load_image(p) for p in req["images"]]
    policy = HyEmbodiedPolicy.from_checkpoint(resolve_checkpoint(config), dtype=model.get("dtype", "fp16"),
                                              prefix_len=int(model.get("prefix_len", 240)), n_cameras=len(images),
                                              norm_stats_path=model.get("norm_stats_path")).to("rpu")
    try:
        out = policy.infer(images=images, instruction=req["instruction"], ee_pose=req.get("ee_pose"), state=req.get("state"),
                           noise_seed=int(req.get("noise_seed", 0)))
        print(f"actions_normalized={tuple(out.actions_normalized.shape)} physical={out.physical_action_available} "
              f"latency_ms={out.latency_ms:.3f}")
    finally:
        policy.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
