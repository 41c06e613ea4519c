#!/usr/bin/env python3
"""Wall-OSS vision-language-action policy: action chunk from camera images, an instruction and proprioception.

The checkpoint directory must hold config.json, the safetensors shards, the Qwen2.5-VL processor files and the
normalizer_action.pth / normalizer_propri.pth sidecars."""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _config import check_execution, load_toml, ok, parse_args, require_model, require_request

FAMILY = "Wall-OSS (Qwen2.5-VL backbone + flow-matching action head)"


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
    prop = req.get("proprioception")
    if not isinstance(prop, list) or not prop or not all(isinstance(v, (int, float)) and not isinstance(v, bool) for v in prop):
        raise ValueError("[request].proprioception must be a non-empty list of numbers")
    if len(req["images"]) != len(model.get("camera_names", ["face_view"])):
        raise ValueError("[request].images needs one path per entry of [model].camera_names")
    check_execution(config, {"prefill", "vision", "action"})
    return config


def main() -> int:
    args = parse_args("wall_oss.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    from _config import load_image, resolve_checkpoint
    from rpu_backend.api import WallOssPolicy
    model, req = config["model"], config["request"]
    images = [load_image(p) for p in req["images"]]
    policy = WallOssPolicy.from_pretrained(
        resolve_checkpoint(config), dataset_key=model.get("dataset_key", "berkeley_autolab_ur5"),
        camera_names=tuple(model.get("camera_names", ["face_view"])), action_horizon=int(model.get("action_horizon", 32)),
        num_steps=int(model.get("num_steps", 10)), max_seq_len=int(model.get("max_seq_len", 2048)),
        rpu_execution=config.get("rpu_execution")).to("rpu")
    try:
        out = policy.infer(images=images, instruction=req["instruction"], proprioception=req["proprioception"],
                           noise_seed=int(req.get("noise_seed", 0)))
    finally:
        policy.close()
    print(f"actions={tuple(out.actions.shape)} action_hz={out.action_hz:g} latency_ms={out.latency_ms:.3f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
