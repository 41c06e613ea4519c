#!/usr/bin/env python3
"""Pi0.5 action-chunk prediction from a saved LeRobot-style batch (``torch.save`` of a dict)."""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _config import check_execution, load_toml, ok, parse_args, require_model, require_request, resolve_checkpoint


def load_config(path) -> dict:
    config = load_toml(path)
    require_model(config)
    req = require_request(config, fields=(("batch_file", str), ("num_steps", int), ("prepare_graphs", bool)))
    if not isinstance(req.get("batch_file"), str):
        raise ValueError("[request].batch_file must be a path string")
    steps = req.get("num_steps", 10)
    if isinstance(steps, bool) or not isinstance(steps, int) or steps < 1:
        raise ValueError("[request].num_steps must be a positive integer")
    check_execution(config, {"prefill", "vision", "action"})
    return config


def main() -> int:
    args = parse_args("pi05.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import time
    import torch
    import rpu_backend  # noqa: F401
    from rpu_backend.api.policy import Pi05Policy

    req = config["request"]
    policy = Pi05Policy.from_pretrained(resolve_checkpoint(config), rpu_execution=config.get("rpu_execution"),
                                        trust_remote_code=False).to("rpu")
    batch = torch.load(Path(req["batch_file"]).expanduser())
    steps = int(req.get("num_steps", 10))
    if req.get("prepare_graphs", False):
        print("prepare_graphs:", policy.prepare_graphs(batch, num_steps=steps))
    t0 = time.perf_counter()
    actions = policy.predict_action_chunk(batch, num_steps=steps)
    torch.cuda.synchronize()
    print(f"actions {tuple(actions.shape)} in {(time.perf_counter() - t0) * 1e3:.2f} ms")
    print(actions[0, :2])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
