#!/usr/bin/env python3
"""Greedy text generation with a dense Qwen3.5 checkpoint (hybrid attention / Gated-DeltaNet decoder)."""
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
    chunk = config.get("rpu_execution", {}).get("prefill", {}).get("chunk_size", "auto")
    if chunk != "auto" and chunk % 64:
        raise ValueError("[rpu_execution.prefill].chunk_size must be 'auto' or a multiple of 64 for Qwen3.5")
    return config


def main() -> int:
    args = parse_args("qwen3_5_0_8b.toml", __doc__)
    config = load_config(args.config)
    if args.check_config:
        return ok(args.config, require_model(config))
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import torch
    from transformers import AutoConfig, AutoModelForCausalLM, AutoTokenizer
    import rpu_backend  # noqa: F401
    from rpu_backend.adapters.qwen3_5 import Qwen3_5Adapter
    from rpu_backend.api.qwen3_5_cache import Qwen3_5Cache

    ckpt = resolve_checkpoint(config)
    local_only = bool(config["model"].get("local_files_only", True))
    hf_config = AutoConfig.from_pretrained(ckpt, local_files_only=local_only, trust_remote_code=False)
    Qwen3_5Adapter.preflight(hf_config)
    tok = AutoTokenizer.from_pretrained(ckpt, local_files_only=local_only, trust_remote_code=False)
    hf_model = AutoModelForCausalLM.from_pretrained(ckpt, dtype=torch.float16, local_files_only=local_only,
                                                    trust_remote_code=False)
    ids = tok(config["generation"]["prompt"], return_tensors="pt").input_ids
    n = config["generation"]["max_new_tokens"]
    L = (ids.shape[1] + n + 64 + 63) // 64 * 64
    model = Qwen3_5Adapter(hf_model, rpu_execution=config.get("rpu_execution")).to_rpu(max_seq_len=L)
    text_config = getattr(hf_config, "text_config", hf_config)
    cache = Qwen3_5Cache.from_config(text_config, max_seq_len=L)
    out = model.generate(ids, past_key_values=cache, max_new_tokens=n, do_sample=False)
    print(tok.decode(out[0, ids.shape[1]:].cpu(), skip_special_tokens=True))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
