#!/usr/bin/env python
"""Same-box baseline for the Pi0.5 action chunk: plain PyTorch eager (cuBLAS GEMMs, cuDNN conv, fused SDPA),
padded/masked formulation, no CUDA graph, none of this repository's kernels or runtime.

    python baseline/eager_pi05.py --batch 1 --steps 20
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from rhinoforge_b200.models.pi05 import Pi05Config, TorchPi05, random_pi05_state_dict  # noqa: E402  (pure PyTorch model)


def run_baseline(batch: int, steps: int, warmup: int, dtype_name: str = "fp16") -> dict:
    """Time `steps` eager chunks of `batch` samples (CUDA events around each chunk); frees its model afterwards."""
    dev = torch.device("cuda", 0)
    dtype = torch.float16 if dtype_name == "fp16" else torch.bfloat16
    cfg = Pi05Config()
    sd = random_pi05_state_dict(cfg, seed=0, std=0.02, dtype=dtype, device=dev)
    m = TorchPi05(cfg, sd, dtype=dtype, device=dev)
    g = torch.Generator().manual_seed(0)
    B = batch
    images = (torch.rand(B, cfg.num_views, 3, 224, 224, generator=g) * 2 - 1).to(dev)
    imask = torch.ones(B, cfg.num_views, dtype=torch.bool)
    tokens = torch.randint(0, cfg.vocab_size, (B, cfg.max_lang_tokens), generator=g)
    tmask = torch.ones(B, cfg.max_lang_tokens, dtype=torch.bool)
    noise = torch.randn(B, cfg.horizon, cfg.action_dim, generator=g).to(dev)
    ms = []
    for i in range(warmup + steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        m.sample_actions(images, imask, tokens, tmask, noise, num_steps=10)
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            ms.append(e0.elapsed_time(e1))
    p50 = statistics.median(ms)
    del m, sd
    torch.cuda.empty_cache()
    return {"impl": "baseline-eager", "metric": "pi05_action_chunk_latency_ms", "value": p50, "unit": "ms",
            "batch": B, "chunks_per_s": B * 1000.0 / p50, "steps": steps, "warmup": warmup, "dtype": dtype_name,
            "data": "synthetic", "config": {"views": cfg.num_views, "seq_len": cfg.max_lang_tokens,
                                            "denoise_steps": 10, "chunk": [cfg.horizon, cfg.action_dim]}}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", default="fp16")
    a = ap.parse_args()
    print(json.dumps(run_baseline(a.batch, a.steps, a.warmup, a.dtype)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
