#!/usr/bin/env python3
"""RhinoVLA through ``RhinoVLAPolicy``: the model repository supplies a runtime factory, this script supplies the
lifecycle (construct -> prepare graphs -> predict) and prints the execution plan the runtime reports back.

``[model].runtime_factory`` names ``module:callable``; the callable receives the checkpoint path, the ``[runtime]``
table as ``config`` and - when ``[rpu_execution]`` is present - the validated execution configuration.  The shipped
configuration points at the stand-in factory below (``rhinovla:demo_runtime_factory``), which implements the whole
handshake without a model, so the script runs end to end on any machine; replace it with the factory your RhinoVLA
integration exports."""
from __future__ import annotations

import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _config import check_execution, load_toml, ok, parse_args, require_request

STAGE_FIELDS = {"prefill": ("chunk_size", "padding_rows", "padding_budget"), "action": ("chunk_size",)}


def load_config(path) -> dict:
    config = load_toml(path)
    model = config.get("model")
    if not isinstance(model, dict) or not isinstance(model.get("checkpoint"), str) or not model["checkpoint"]:
        raise ValueError("[model].checkpoint must be a non-empty string")
    factory = model.get("runtime_factory")
    if not isinstance(factory, str) or factory.count(":") != 1 or not all(factory.split(":")):
        raise ValueError("[model].runtime_factory must use module:callable syntax")
    if "runtime" in config and not isinstance(config["runtime"], dict):
        raise ValueError("[runtime] must be a table")
    req = require_request(config, fields=(("instruction", str), ("request_json", str)))
    if "request_json" not in req and not isinstance(req.get("instruction"), str):
        raise ValueError("[request] needs request_json (a file holding the request object) or an inline instruction")
    check_execution(config, set(STAGE_FIELDS))
    return config


class _DemoRuntime:
    """Stands in for a model-repository runtime: honours the execution request and publishes what it resolved."""

    _rpu_execution_capabilities = STAGE_FIELDS

    def __init__(self, checkpoint, config, rpu_execution):
        self.checkpoint, self.config = checkpoint, dict(config or {})
        if rpu_execution is not None:
            self._rpu_execution = rpu_execution
        self._rpu_execution_resolved_generation = 0

    def _asked(self, stage: str, field: str, default: int) -> int:
        value = dict(getattr(self, "_rpu_execution", {}).get(stage, {})).get(field)
        return value if isinstance(value, int) else default

    def _publish(self, prompt_rows: int) -> None:
        align = 16
        pad = self._asked("prefill", "padding_rows", (-prompt_rows) % align)
        horizon = int(self.config.get("action_horizon", 32))
        self._rpu_execution_resolved = {
            "prefill": {"logical_len": prompt_rows, "execution_len": prompt_rows + pad, "padding_rows": pad,
                        "chunk_size": self._asked("prefill", "chunk_size", 256),
                        "execution_alignment": align if (prompt_rows + pad) % align == 0 else 1},
            "action": {"logical_len": horizon, "execution_len": horizon, "padding_rows": 0,
                       "chunk_size": self._asked("action", "chunk_size", 64)}}
        self._rpu_execution_resolved_generation += 1

    def prepare_graphs(self, **request):
        self._publish(len(str(request.get("instruction", "")).split()) + 2)
        return None

    def predict(self, **request):
        self._publish(len(str(request.get("instruction", "")).split()) + 2)
        horizon, dim = int(self.config.get("action_horizon", 32)), int(self.config.get("action_dim", 7))
        return [[0.0] * dim for _ in range(horizon)]


def demo_runtime_factory(checkpoint, *, config=None, rpu_execution=None):
    return _DemoRuntime(checkpoint, config, rpu_execution)


demo_runtime_factory._rpu_execution_capabilities = STAGE_FIELDS


def main() -> int:
    args = parse_args("rhinovla.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, config["model"]["checkpoint"])
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    from rpu_backend.api import RhinoVLAPolicy
    req = dict(config["request"])
    if "request_json" in req:
        path = Path(req.pop("request_json")).expanduser()
        if not path.is_file():
            raise SystemExit(f"RhinoVLA request JSON not found: {path}")
        loaded = json.loads(path.read_text(encoding="utf-8"))
        if not isinstance(loaded, dict):
            raise SystemExit("RhinoVLA request JSON must contain an object")
        req.update(loaded)
    kwargs = {"config": config["runtime"]} if config.get("runtime") else {}
    policy = RhinoVLAPolicy.from_pretrained(config["model"]["checkpoint"], runtime_factory=config["model"]["runtime_factory"],
                                            rpu_execution=config.get("rpu_execution"), **kwargs)
    policy.prepare_graphs(**req)
    out = policy.predict(**req)
    shape = getattr(out, "shape", None) or (len(out), len(out[0]) if out and hasattr(out[0], "__len__") else None)
    print(f"output_type={type(out).__name__} shape={tuple(shape)}")
    for stage, plan in policy.last_rpu_execution_plan.items():
        print(f"  {stage}: {plan}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
