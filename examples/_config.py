"""Standard-library-only helpers shared by the example scripts: TOML loading and validation run
before torch or the backend is imported, so ``--check-config`` works on any machine."""
from __future__ import annotations

import argparse
import tomllib
from pathlib import Path

CONFIG_DIR = Path(__file__).with_name("configs")
_STAGES = {"prefill", "vision", "action"}
_FIELDS = {"chunk_size", "padding_rows", "padding_budget"}


def parse_args(default_config: str, description: str) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--config", type=Path, default=CONFIG_DIR / default_config)
    ap.add_argument("--check-config", action="store_true", help="validate the TOML file and exit")
    return ap.parse_args()


def load_toml(path: Path) -> dict:
    with Path(path).open("rb") as f:
        return tomllib.load(f)


def require_model(config: dict) -> str:
    model = config.get("model")
    if not isinstance(model, dict) or not (model.get("alias") or model.get("checkpoint")):
        raise ValueError("[model] needs alias or checkpoint")
    return model.get("checkpoint") or model["alias"]


def require_generation(config: dict) -> None:
    gen = config.get("generation")
    if not isinstance(gen, dict) or not isinstance(gen.get("prompt"), str):
        raise ValueError("[generation].prompt must be a string")
    n = gen.get("max_new_tokens")
    if not isinstance(n, int) or isinstance(n, bool) or n < 1:
        raise ValueError("[generation].max_new_tokens must be a positive integer")


def check_execution(config: dict, supported_stages) -> None:
    """Shape check of ``[rpu_execution.<stage>]`` without importing the backend."""
    ex = config.get("rpu_execution", {})
    if not isinstance(ex, dict):
        raise ValueError("[rpu_execution] must be a table")
    for stage, fields in ex.items():
        if stage not in _STAGES:
            raise ValueError(f"[rpu_execution.{stage}] is not a known stage")
        if stage not in supported_stages:
            raise ValueError(f"[rpu_execution.{stage}] is not supported by this model entry point")
        for k, v in fields.items():
            if k not in _FIELDS:
                raise ValueError(f"[rpu_execution.{stage}].{k} is not a known field")
            if k == "chunk_size" and v != "auto" and (not isinstance(v, int) or v <= 0 or v % 16):
                raise ValueError(f"[rpu_execution.{stage}].chunk_size must be 'auto' or a positive multiple of 16")


def resolve_checkpoint(config: dict) -> str:
    from rpu_backend.model_registry import model_path
    m = config["model"]
    return m.get("checkpoint") or str(model_path(m["alias"]))


def ok(path, location) -> int:
    print(f"configuration OK: {path} ({location})")
    return 0


def require_request(config: dict, *, image: bool = False, fields=()) -> dict:
    req = config.get("request")
    if not isinstance(req, dict):
        raise ValueError("configuration needs a [request] table")
    if image and not isinstance(req.get("image"), str):
        raise ValueError("[request].image must be a path string")
    for name, kind in fields:
        if name in req and (not isinstance(req[name], kind) or isinstance(req[name], bool) and kind is int):
            raise ValueError(f"[request].{name} must be of type {kind.__name__}")
    return req


def load_image(path: str):
    """RGB float tensor ``[3, H, W]`` in [0, 1] from an image file (PIL) or a ``.pt``/``.npy`` array."""
    import torch
    p = Path(path).expanduser()
    if p.suffix == ".pt":
        return torch.load(p).float()
    if p.suffix == ".npy":
        import numpy as np
        return torch.from_numpy(np.load(p)).float()
    from PIL import Image
    import numpy as np
    arr = np.asarray(Image.open(p).convert("RGB"), dtype="float32") / 255.0
    return torch.from_numpy(arr).permute(2, 0, 1)
