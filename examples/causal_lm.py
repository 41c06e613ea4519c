#!/usr/bin/env python3
"""Greedy text generation with a supported Qwen3 or Llama checkpoint."""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _config import check_execution, load_toml, ok, parse_args, require_generation, require_model, resolve_checkpoint


def load_config(path) -> dict:
    config = load_toml(path)
    require_model(config)
    require_generation(config)
    check_execution(config, {"prefill"})
    return config


def main() -> int:
    args = parse_args("qwen3_0_6b.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import torch
    from transformers import AutoTokenizer
    from rpu_backend import RPUCache, RPUModelForCausalLM

    ckpt = resolve_checkpoint(config)
    local_only = bool(config["model"].get("local_files_only", True))
    tok = AutoTokenizer.from_pretrained(ckpt, local_files_only=local_only, trust_remote_code=False)
    model = RPUModelForCausalLM.from_pretrained(ckpt, dtype=torch.float16, device="rpu",
                                                rpu_execution=config.get("rpu_execution"),
                                                local_files_only=local_only, trust_remote_code=False)
    inputs = tok(config["generation"]["prompt"], return_tensors="pt")
    n = config["generation"]["max_new_tokens"]
    cache = RPUCache.from_model(model, input_ids=inputs.input_ids, max_new_tokens=n)
    from rpu_backend.runtime.control import warmup_iters
    for _ in range(warmup_iters()):          # RPU_WARMUP untimed runs (graph capture, allocator warm-up) before the real one
        model.generate(inputs.input_ids, past_key_values=cache, max_new_tokens=n, do_sample=False, use_cache=True)
        cache.reset()
    out = model.generate(inputs.input_ids, past_key_values=cache, max_new_tokens=n, do_sample=False, use_cache=True)
    print(tok.decode(out[0, inputs.input_ids.shape[1]:].cpu(), skip_special_tokens=True))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
