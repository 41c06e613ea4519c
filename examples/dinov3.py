#!/usr/bin/env python3
"""DINOv3 ViT-B/16 image features: last hidden state and the CLS pooled vector."""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _config import check_execution, load_image, load_toml, ok, parse_args, require_model, require_request, resolve_checkpoint


def load_config(path) -> dict:
    config = load_toml(path)
    require_model(config)
    require_request(config, image=True)
    check_execution(config, {"vision"})
    return config


def main() -> int:
    args = parse_args("dinov3_vitb16.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import torch
    from transformers import AutoConfig, AutoModel
    import rpu_backend  # noqa: F401
    from rpu_backend.adapters.dinov3 import DINOv3Adapter

    ckpt = resolve_checkpoint(config)
    local_only = bool(config["model"].get("local_files_only", True))
    hf_config = AutoConfig.from_pretrained(ckpt, local_files_only=local_only, trust_remote_code=False)
    DINOv3Adapter.preflight(hf_config)                       # config-only rejection before any weight is read
    hf_model = AutoModel.from_pretrained(ckpt, dtype=torch.float16, local_files_only=local_only, trust_remote_code=False)
    model = DINOv3Adapter(hf_model, rpu_execution=config.get("rpu_execution")).to_rpu()
    img = load_image(config["request"]["image"])
    size = hf_config.image_size
    img = torch.nn.functional.interpolate(img[None], size=(size, size), mode="bilinear", align_corners=False)
    mean = torch.tensor([0.485, 0.456, 0.406]).view(1, 3, 1, 1)
    std = torch.tensor([0.229, 0.224, 0.225]).view(1, 3, 1, 1)
    out = model((img - mean) / std)
    print("last_hidden_state", tuple(out.last_hidden_state.shape), "pooler_output", tuple(out.pooler_output.shape))
    print("cls[:8] =", [round(float(v), 4) for v in out.pooler_output[0, :8]])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
