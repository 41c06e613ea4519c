#!/usr/bin/env python
"""Headline benchmark: Qwen3-8B-architecture greedy decode throughput (tokens/s) on N B200s.

    python bench.py --gpus 1 --steps 256 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload (the reference's serving protocol, docs/performance.md:12-64): batch B uniform-random
prompts of 1024 tokens, paged KV with 16-token pages, tensor parallelism over the N GPUs, the
whole decode step replayed from one CUDA graph.  Random-init weights (normal std 0.02, seed 0),
synthetic token ids.  One "step" = one decode step of the whole batch.  Timed on the device
with CUDA events, max over ranks; rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--quant", default=None, choices=[None, "w8a16"])
    ap.add_argument("--sweep", default="", help="extra batch sizes to report, e.g. 1,8,32")
    ap.add_argument("--ttft-samples", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true", help="launch decode steps eagerly (kernel profiling only)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    return ap.parse_args(argv)


REFERENCE_UNAVAILABLE = ("reference needs the restricted 'rhino_launch 1.0.0' CMake package, the rhinoOpLib operator "
                         "asset and an RPU board; pip install of /root/reference fails at CMake configure")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def run(args) -> dict:
    import torch
    from rhinoforge_b200 import _native as N
    from rhinoforge_b200.models.decoder import PROFILES
    from rhinoforge_b200.parallel.tp import TPContext
    from rhinoforge_b200.runtime.engine import DecoderEngine, random_weight_getter

    tp = TPContext.from_env()
    if tp.world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={tp.world}: launch with torch.distributed.run")
    dev = tp.device
    torch.cuda.set_device(dev)
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    cfg = PROFILES[args.model]
    batches = sorted({args.batch, *[int(b) for b in args.sweep.split(",") if b]})
    max_b = max(batches)
    max_seq = args.prompt_len + args.steps * 2 + args.warmup + 64
    t0 = time.time()
    eng = DecoderEngine(cfg, random_weight_getter(cfg, seed=0, std=0.02, dtype=dtype, device=dev), dtype=dtype,
                        max_batch=max_b, max_seq_len=max_seq, max_prefill_tokens=8192,
                        tp=tp, quant=args.quant)
    torch.cuda.synchronize()
    startup_s = time.time() - t0
    lib = N.lib()
    lib.rf_launch_count.restype = __import__("ctypes").c_uint64
    gen = torch.Generator().manual_seed(0)
    results = {}
    headline = None
    for B in batches:
        prompts = [torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=gen) for _ in range(B)]
        # ---- TTFT: prefill + first token, device-timed, median of samples
        ttfts = []
        for _ in range(max(1, args.ttft_samples)):
            tp.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.prefill(prompts)
            e1.record(); torch.cuda.synchronize()
            ttfts.append(tp.max_float(e0.elapsed_time(e1)))
        # ---- decode: BUILD the graph once, warm up, then time K replays
        c0 = lib.rf_launch_count()
        eng.capture(B)
        per_step_launches = (lib.rf_launch_count() - c0) // 2   # one eager + one captured step
        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        eng.decode(args.warmup)
        tp.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g = eng.graphs[B]
        if args.profiler_range:
            torch.cuda.profiler.start()
        for _ in range(args.steps):
            if args.no_graph:
                eng._decode_step(B)
            else:
                g.replay()
        if args.profiler_range:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        e1.record()
        tp.barrier(); torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = tp.max_float(e0.elapsed_time(e1)) / args.steps
        eng.advance_lengths(args.steps)
        eng.check_status()
        # ---- end to end through the host-driven step API: per step H2D of the input ids from pinned
        # memory, graph replay, D2H of the produced ids, host sync
        eng.prefill(prompts)
        h_in = torch.zeros(B, dtype=torch.int32).pin_memory()
        h_out = torch.zeros(B, dtype=torch.int32).pin_memory()
        h_in.copy_(eng.ids[:B].cpu())
        for _ in range(args.warmup):
            eng.step_from_host(h_in, h_out); torch.cuda.synchronize(); h_in.copy_(h_out)
        tp.barrier(); torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(args.steps):
            eng.step_from_host(h_in, h_out)
            torch.cuda.synchronize()
            h_in.copy_(h_out)
        e2e_s = tp.max_float(time.perf_counter() - t1)
        eng.check_status()
        res = {"batch": B, "tok_s": B * 1000.0 / ms, "ms_per_step": ms, "ttft_ms_p50": statistics.median(ttfts),
               "e2e_tok_s": B * args.steps / e2e_s, "launches_per_step": int(per_step_launches), "clocks": clocks}
        results[B] = res
        if B == args.batch:
            headline = res
    wbytes = eng.weight_bytes()
    eng.close()
    B = args.batch
    out = {
        "metric": "decode_tokens_per_s", "value": headline["tok_s"], "unit": "tokens/s", "n_gpus": tp.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": headline["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": args.dtype if not args.quant else f"{args.dtype}+int8w", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"{cfg.name}-architecture random-init (std 0.02, seed 0)", "global_batch": B,
                   "seq_len": args.prompt_len, "decode_steps": args.steps, "parallelism": f"tp{tp.world}",
                   "kv": "paged, 16-token pages", "graph": "whole decode step in one CUDA graph",
                   "l2": f"inputs larger than L2: {wbytes / 1e9:.1f} GB of weights per GPU read every step"},
        "clocks": headline["clocks"],
        "e2e": {"value": headline["e2e_tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * B},
        "gpu_launches": headline["launches_per_step"] * args.steps,
        "ttft_ms_p50": headline["ttft_ms_p50"],
        "startup_s": startup_s,
        "by_batch": {str(b): {k: v for k, v in r.items() if k != "clocks"} for b, r in results.items()},
    }
    return out if tp.rank == 0 else None


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    out = run(args)
    if out is not None:
        print(json.dumps(out))
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
