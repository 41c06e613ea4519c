#!/usr/bin/env python3
"""Qwen2.5-VL vision tower on one image: merged patch embeddings (window attention, full-attention blocks in between)."""
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
    args = parse_args("qwen25_vl_vision.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import torch
    from transformers import AutoConfig, AutoModelForImageTextToText
    import rpu_backend  # noqa: F401
    from rpu_backend.adapters.qwen25_vl_vision import Qwen25VLVisionAdapter

    ckpt = resolve_checkpoint(config)
    local_only = bool(config["model"].get("local_files_only", True))
    hf_config = AutoConfig.from_pretrained(ckpt, local_files_only=local_only, trust_remote_code=False)
    Qwen25VLVisionAdapter.preflight(hf_config)               # config-only rejection before any weight is read
    hf_model = AutoModelForImageTextToText.from_pretrained(ckpt, dtype=torch.float16, local_files_only=local_only,
                                                           trust_remote_code=False)
    visual = hf_model.model.visual if hasattr(hf_model, "model") else hf_model.visual
    tower = Qwen25VLVisionAdapter(visual, rpu_execution=config.get("rpu_execution")).to_rpu()
    vc = visual.config
    unit = vc.patch_size * vc.spatial_merge_size
    img = load_image(config["request"]["image"])
    side = max(unit, min(img.shape[-2:]) // unit * unit)
    img = torch.nn.functional.interpolate(img[None], size=(side, side), mode="bilinear", align_corners=False)[0]
    g, p, m = side // vc.patch_size, vc.patch_size, vc.spatial_merge_size
    # processor layout: [T, C * temporal * p * p] rows in merge-block order, the frame repeated over the temporal patch
    x = img.view(3, g // m, m, p, g // m, m, p).permute(1, 4, 2, 5, 0, 3, 6).reshape(g * g, 3, 1, p, p)
    x = x.expand(-1, -1, vc.temporal_patch_size, -1, -1).reshape(g * g, -1)
    emb = tower(x, torch.tensor([[1, g, g]]))
    print("image_embeds", tuple(emb.shape), "first row[:8] =", [round(float(v), 4) for v in emb[0, :8]])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
