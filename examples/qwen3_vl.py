#!/usr/bin/env python3
"""Image + text greedy generation with Qwen3-VL (manual decode loop over the model's forward)."""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _config import check_execution, load_toml, ok, parse_args, require_model, require_request, resolve_checkpoint


def load_config(path) -> dict:
    config = load_toml(path)
    require_model(config)
    req = require_request(config, image=True, fields=(("prompt", str), ("max_new_tokens", int)))
    if not isinstance(req.get("prompt"), str):
        raise ValueError("[request].prompt must be a string")
    if not isinstance(req.get("max_new_tokens", 32), int) or req.get("max_new_tokens", 32) < 1:
        raise ValueError("[request].max_new_tokens must be a positive integer")
    check_execution(config, {"prefill", "vision"})
    return config


def main() -> int:
    args = parse_args("qwen3_vl_2b.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import torch
    from PIL import Image
    from transformers import AutoProcessor
    from rpu_backend import RPUCache
    from rpu_backend.api.conditional_generation import RPUModelForConditionalGeneration

    ckpt = resolve_checkpoint(config)
    req = config["request"]
    local_only = bool(config["model"].get("local_files_only", True))
    proc = AutoProcessor.from_pretrained(ckpt, local_files_only=local_only, trust_remote_code=False)
    model = RPUModelForConditionalGeneration.from_pretrained(ckpt, dtype=torch.float16, device="rpu",
                                                             rpu_execution=config.get("rpu_execution"),
                                                             local_files_only=local_only, trust_remote_code=False)
    messages = [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": req["prompt"]}]}]
    text = proc.apply_chat_template(messages, add_generation_prompt=True)
    inputs = proc(text=[text], images=[Image.open(Path(req["image"]).expanduser()).convert("RGB")], return_tensors="pt")
    n = int(req.get("max_new_tokens", 32))
    cache = RPUCache.from_model(model.model.language_model, input_ids=inputs.input_ids, max_new_tokens=n)
    o = model(input_ids=inputs.input_ids, past_key_values=cache, logits_to_keep=1, use_cache=True, return_dict=True,
              attention_mask=inputs.attention_mask, pixel_values=inputs.pixel_values, image_grid_thw=inputs.image_grid_thw)
    eos = proc.tokenizer.eos_token_id
    out = []
    for _ in range(n):
        nxt = int(o.logits[0, -1].argmax())
        if nxt == eos:
            break
        out.append(nxt)
        o = model(input_ids=torch.tensor([[nxt]]), past_key_values=cache, logits_to_keep=1, use_cache=True, return_dict=True)
    print(proc.tokenizer.decode(out, skip_special_tokens=True))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
