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
    ap.add_argument("--workload", default="decode", choices=["decode", "pi05", "qwen3vl"],
                    help="decode: causal-LM decode throughput (headline); pi05: action-chunk latency; "
                         "qwen3vl: multimodal prefill + decode")
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--quant", default=None, choices=[None, "w8a16"])
    ap.add_argument("--sweep", default="1,8,32", help="extra batch sizes reported in by_batch ('' = only --batch)")
    ap.add_argument("--no-baseline", action="store_true",
                    help="skip the same-box PyTorch eager (+NCCL) baseline run that fills vs_baseline")
    ap.add_argument("--no-tokens-check", action="store_true",
                    help="skip the greedy-token check of a 4-layer truncation against the fp32 oracle / the TP=1 engine")
    ap.add_argument("--ttft-samples", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true", help="launch decode steps eagerly (kernel profiling only)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    return ap.parse_args(argv)


REFERENCE_UNAVAILABLE = ("reference needs the restricted 'rhino_launch 1.0.0' CMake package, the rhinoOpLib operator "
                         "asset and an RPU board; pip install of the reference source fails at CMake configure")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines, self.first = index, None, [], 0

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

    def wait_first(self, timeout_s: float = 8.0) -> None:
        """Block until the first sample has arrived (nvidia-smi takes a while to start on an 8-GPU box), so that a
        short timed region is not over before sampling begins."""
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < timeout_s:
            time.sleep(0.01)

    def mark(self) -> None:
        """Start of the timed region: only samples taken from here on are reported."""
        self.first = len(self.lines)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        lines = self.lines[self.first:]
        if len(lines) < 2:       # region shorter than two sampling periods: include the warm-up samples just before it
            lines = self.lines[max(0, self.first - 4):]
        for ln in lines:
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


def tokens_check(args, tp, dtype) -> dict:
    """Correctness bit of the benchmarked configuration: a 4-layer truncation of the benchmarked model (same widths,
    same random weights, same tensor-parallel degree, same kernels and graph path) decodes 16 greedy tokens for 4
    prompts of 64 tokens; rank 0 compares them with (a) the plain-PyTorch fp32 forward of the same weights - tokens
    must agree until the oracle's own top-2 margin is inside 16-bit noise, after which sequences legitimately part
    ways - and, under tensor parallelism, (b) a TP=1 engine on rank 0 (exact match count reported)."""
    import dataclasses
    import torch
    from rhinoforge_b200.models.decoder import PROFILES, TorchDecoder
    from rhinoforge_b200.parallel.tp import TPContext
    from rhinoforge_b200.runtime.engine import DecoderEngine, random_weight_getter
    cfg = dataclasses.replace(PROFILES[args.model], num_layers=4, name=PROFILES[args.model].name + "-4layer")
    dev = tp.device
    get = random_weight_getter(cfg, seed=0, std=0.02, dtype=dtype, device=dev)
    gen = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab_size, (64,), generator=gen) for _ in range(4)]
    n_new = 16
    eng = DecoderEngine(cfg, get, dtype=dtype, max_batch=4, max_seq_len=128, max_prefill_tokens=512, tp=tp,
                        quant=args.quant)
    toks = eng.generate(prompts, n_new).cpu()
    eng.close()
    out = {"layers": 4, "prompts": 4, "new_tokens": n_new}
    if tp.rank == 0:
        if args.quant is None:
            from rhinoforge_b200.models.decoder import weight_shapes
            sd = {name: get(name) for name, _, _ in weight_shapes(cfg)}
            oracle = TorchDecoder(cfg, sd, dtype=torch.float32, device=dev)
            agree, compared = True, 0
            for b, p in enumerate(prompts):
                oracle.reset()
                rt, rl = oracle.greedy(p[None].to(dev), n_new)
                for t in range(n_new):
                    compared += 1
                    if int(toks[b, t]) != int(rt[0, t]):
                        lg = rl[0, t].float()
                        margin = float(lg[int(rt[0, t])] - lg[int(toks[b, t])])
                        out.setdefault("first_mismatches", []).append({"seq": b, "step": t, "margin": margin})
                        agree &= margin < 0.02
                        break
            del oracle, sd
            out.update({"vs_fp32_oracle": bool(agree), "oracle_tokens_compared": compared})
        if tp.enabled:
            e1 = DecoderEngine(cfg, get, device=dev, dtype=dtype, max_batch=4, max_seq_len=128, max_prefill_tokens=512,
                               tp=TPContext.single(dev), quant=args.quant)
            t1 = e1.generate(prompts, n_new).cpu()
            e1.close()
            out["tp1_equal_tokens"] = f"{int((t1 == toks).sum())}/{t1.numel()}"
            out["vs_tp1_engine"] = bool((t1 == toks).all())
        out["ok"] = bool(out.get("vs_fp32_oracle", True) and (out.get("vs_tp1_engine", True) or out.get("vs_fp32_oracle", False)))
    torch.cuda.empty_cache()
    tp.barrier()
    return out


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
        eng.reserve_steps(args.steps)             # KV pages for the raw graph replays below
        sampler.wait_first()
        tp.barrier(); torch.cuda.synchronize()
        sampler.mark()
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
    del eng
    torch.cuda.empty_cache()
    B = args.batch
    check = None if args.no_tokens_check else tokens_check(args, tp, dtype)
    # ---- same-box baseline: the same model in plain PyTorch eager (cuBLAS, SDPA, NCCL all-reduce), same batch, prompt
    # length, steps and warm-up; on one GPU additionally with its decode step captured in a CUDA graph (the stronger
    # baseline, used for vs_baseline there; NCCL collectives inside a graph capture did not return on this pool).
    base = None
    if not args.no_baseline:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
        from eager_tp import run_baseline
        eager = run_baseline(args.model, B, args.prompt_len, args.steps, args.warmup, args.dtype, cuda_graph=False)
        base = {"impl": eager["impl"], "decode_tok_s": eager["value"], "ms_per_step": eager["ms_per_step"],
                "ttft_ms_p50": eager["ttft_ms_p50"]}
        if tp.world == 1:
            graphed = run_baseline(args.model, B, args.prompt_len, args.steps, args.warmup, args.dtype, cuda_graph=True)
            base.update({"impl": graphed["impl"], "decode_tok_s": graphed["value"], "ms_per_step": graphed["ms_per_step"],
                         "eager_decode_tok_s": eager["value"], "eager_ms_per_step": eager["ms_per_step"]})
        base["ttft_speedup"] = base["ttft_ms_p50"] / headline["ttft_ms_p50"]
    out = {
        "metric": "decode_tokens_per_s", "value": headline["tok_s"], "unit": "tokens/s", "n_gpus": tp.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": headline["ms_per_step"],
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": (headline["tok_s"] / base["decode_tok_s"]) if base else None,
        "baseline": base, "tokens_check": (check or {}).get("ok") if tp.rank == 0 else None,
        "tokens_check_detail": check,
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


def _timed(fn, steps: int, warmup: int):
    """(per-call device ms list, clocks): CUDA events around every call, clocks sampled meanwhile."""
    import torch
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    sampler.wait_first()
    sampler.mark()
    ms = []
    for _ in range(steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    return ms, sampler.stop()


def run_pi05(args) -> dict:
    """Pi0.5-architecture action chunk: 3 views of 224x224, 200 prompt tokens, 10 Euler steps, chunk 50x32.
    A "step" is one full chunk (vision + prefix prefill + denoise loop)."""
    import ctypes
    import torch
    from rhinoforge_b200 import _native as N
    from rhinoforge_b200.models.pi05 import Pi05Config, Pi05Engine, random_pi05_state_dict
    if args.gpus != 1:
        raise SystemExit("the pi05 workload runs on one GPU")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    cfg = Pi05Config()
    batches = sorted({1, *[int(b) for b in args.sweep.split(",") if b]})
    t0 = time.time()
    sd = random_pi05_state_dict(cfg, seed=0, std=0.02, dtype=dtype, device=dev)
    eng = Pi05Engine(cfg, sd, dtype=dtype, max_batch=max(batches))
    del sd
    torch.cuda.synchronize()
    startup_s = time.time() - t0
    lib = N.lib()
    lib.rf_launch_count.restype = ctypes.c_uint64
    g = torch.Generator().manual_seed(0)
    res = {}
    for B in batches:
        images = torch.rand(B, cfg.num_views, 3, 224, 224, generator=g).mul_(2).sub_(1).pin_memory()
        imask = torch.ones(B, cfg.num_views, dtype=torch.bool)
        tokens = torch.randint(0, cfg.vocab_size, (B, cfg.max_lang_tokens), generator=g).pin_memory()
        tmask = torch.ones(B, cfg.max_lang_tokens, dtype=torch.bool)
        noise = torch.randn(B, cfg.horizon, cfg.action_dim, generator=g).pin_memory()
        d_img, d_noise = images.to(dev), noise.to(dev)
        host_out = torch.empty(B, cfg.horizon, cfg.action_dim, dtype=dtype).pin_memory()

        def device_only():
            eng.predict(d_img, imask, tokens, tmask, d_noise, num_steps=10)

        def end_to_end():           # inputs from pinned host memory every call, actions read back
            out = eng.predict(images.to(dev, non_blocking=True), imask, tokens, tmask, noise.to(dev, non_blocking=True),
                              num_steps=10)
            host_out.copy_(out, non_blocking=True)
            torch.cuda.synchronize()

        device_only()               # BUILD
        c0 = lib.rf_launch_count()
        eng.predict(d_img, imask, tokens, tmask, d_noise, num_steps=10, use_graph=False)
        chunk_launches = lib.rf_launch_count() - c0       # kernels of one chunk, launched one by one
        c0 = lib.rf_launch_count()
        device_only()
        eager_launches = lib.rf_launch_count() - c0       # kernels launched outside the two graphs on a replay
        ms, clocks = _timed(device_only, args.steps, max(args.warmup, 3))
        t1 = time.perf_counter()
        for _ in range(args.steps):
            end_to_end()
        e2e_ms = (time.perf_counter() - t1) * 1000.0 / args.steps
        eng.check_status()
        # where the time goes: vision tower, prefix (rest of prefill), denoise loop
        def vision_only():
            eng.vision(d_img.flatten(0, 1))
        lens = eng.prefill(d_img, imask, tokens, tmask)
        v_ms, _ = _timed(vision_only, 5, 2)
        p_ms, _ = _timed(lambda: eng.prefill(d_img, imask, tokens, tmask), 5, 2)
        d_ms, _ = _timed(lambda: eng.denoise(lens, d_noise, 10), 5, 2)
        if args.profiler_range:
            torch.cuda.profiler.start()
            eng.predict(d_img, imask, tokens, tmask, d_noise, num_steps=10, use_graph=not args.no_graph)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        parts = {"vision_ms": statistics.median(v_ms), "prefill_ms": statistics.median(p_ms),
                 "denoise_ms": statistics.median(d_ms)}
        res[B] = {"batch": B, **parts, "ms_p50": statistics.median(ms), "ms_p90": sorted(ms)[int(0.9 * (len(ms) - 1))],
                  "chunks_per_s": B * 1000.0 / statistics.median(ms), "e2e_ms": e2e_ms,
                  "launches_outside_graph": int(eager_launches), "launches_per_chunk": int(chunk_launches), "clocks": clocks,
                  "h2d": images.numel() * 4 + tokens.numel() * 8 + noise.numel() * 4, "d2h": host_out.numel() * 2}
    eng.close()
    del eng
    torch.cuda.empty_cache()
    h = res[1]
    base = None
    if not args.no_baseline:
        # same box, same inputs: PyTorch eager (cuBLAS, cuDNN, fused SDPA), padded / masked formulation, no graph
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
        from eager_pi05 import run_baseline as eager_pi05
        base = {str(b): eager_pi05(b, min(args.steps, 10), 3, args.dtype) for b in batches}
        for b, r in res.items():
            r["baseline_eager_ms"] = base[str(b)]["value"]
            r["speedup_vs_eager"] = base[str(b)]["value"] / r["ms_p50"]
    return {
        "baseline": None if base is None else {"impl": "PyTorch eager on the same GPU (baseline/eager_pi05.py)",
                                               "ms_by_batch": {b: r["value"] for b, r in base.items()}},
        "metric": "pi05_action_chunk_latency_ms", "value": h["ms_p50"], "unit": "ms", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": h["ms_p50"], "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None if base is None else base["1"]["value"] / h["ms_p50"], "dtype": args.dtype, "data": "synthetic",
        "impl": "ours",
        "config": {"model": "pi0.5-architecture random-init (std 0.02, seed 0): SigLIP-So400m/14 + Gemma-2B + Gemma-300M expert",
                   "global_batch": 1, "views": cfg.num_views, "image": "224x224", "seq_len": cfg.max_lang_tokens,
                   "denoise_steps": 10, "chunk": [cfg.horizon, cfg.action_dim], "parallelism": "tp1",
                   "graph": "vision tower + prefix prefill in one CUDA graph, denoise loop in another",
                   "l2": "inputs larger than L2: ~6.7 GB of weights read per chunk"},
        "clocks": h["clocks"], "p90_ms": h["ms_p90"],
        "e2e": {"value": h["e2e_ms"], "unit": "ms", "h2d_bytes_per_step": h["h2d"], "d2h_bytes_per_step": h["d2h"]},
        "gpu_launches": h["launches_per_chunk"] * args.steps,      # kernels of this library replayed from the two graphs
        "startup_s": startup_s,
        "by_batch": {str(b): {k: v for k, v in r.items() if k != "clocks"} for b, r in res.items()},
    }


def run_qwen3vl(args) -> dict:
    """Qwen3-VL-2B-architecture: batch 4, every sample 2 images (448x448 -> 28x28 patches each) + 256 text tokens;
    reports multimodal prefill ms (vision tower + text prefill with DeepStack) and greedy decode tokens/s."""
    import ctypes
    import torch
    from rhinoforge_b200 import _native as N
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLConfig
    from rhinoforge_b200.models.decoder import PROFILES, weight_shapes
    from rhinoforge_b200.models.qwen3_vl import Qwen3VLEngine
    if args.gpus != 1:
        raise SystemExit("the qwen3vl workload runs on one GPU")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    tc = PROFILES["qwen3-vl-2b-text"]
    hf = Qwen3VLConfig(
        text_config=dict(hidden_size=tc.hidden_size, intermediate_size=tc.intermediate_size, num_hidden_layers=tc.num_layers,
                         num_attention_heads=tc.num_heads, num_key_value_heads=tc.num_kv_heads, head_dim=tc.head_dim,
                         vocab_size=tc.vocab_size, max_position_embeddings=4096, tie_word_embeddings=True,
                         rope_parameters={"rope_type": "default", "rope_theta": tc.rope_theta,
                                          "mrope_section": list(tc.mrope_section), "mrope_interleaved": True}),
        vision_config=dict(depth=24, hidden_size=1024, num_heads=16, intermediate_size=4096, out_hidden_size=tc.hidden_size,
                           num_position_embeddings=2304, deepstack_visual_indexes=[5, 11, 17]),
        tie_word_embeddings=True)
    gen = torch.Generator(device=dev).manual_seed(0)
    cache = {}

    def get(name: str) -> torch.Tensor:          # random weights drawn on the device by name
        if name not in cache:
            cache[name] = shape_of[name]()
        return cache[name]
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLForConditionalGeneration
    with torch.device("meta"):
        skeleton = Qwen3VLForConditionalGeneration(hf)
    shape_of = {}
    for n, p in skeleton.state_dict().items():
        shp = tuple(p.shape)
        if p.dim() >= 2:
            shape_of[n] = (lambda s=shp: (torch.randn(s, generator=gen, device=dev) * 0.02).to(dtype))
        elif "norm" in n and n.endswith("weight"):
            shape_of[n] = (lambda s=shp: torch.ones(s, device=dev, dtype=dtype))
        else:
            shape_of[n] = (lambda s=shp: torch.zeros(s, device=dev, dtype=dtype))
    t0 = time.time()
    BATCH = 4
    eng = Qwen3VLEngine(hf, get, names=set(shape_of), dtype=dtype, max_seq_len=2048, max_batch=BATCH,
                        max_patches=BATCH * 2 * 28 * 28, max_prefill_tokens=BATCH * 1024)
    cache.clear()
    torch.cuda.synchronize()
    startup_s = time.time() - t0
    grid = torch.tensor([[1, 28, 28], [1, 28, 28]])
    n_img = 2 * (28 * 28 // 4)
    g = torch.Generator().manual_seed(0)
    text = torch.randint(0, 150000, (256,), generator=g)
    ids = torch.cat((text[:8], torch.full((n_img // 2,), eng.image_token_id), text[8:16],
                     torch.full((n_img // 2,), eng.image_token_id), text[16:]))
    # uniform [0,1] pixels normalised with mean/std 0.5, one pinned host tensor per sample
    pxs = [torch.rand(2 * 28 * 28, 3 * 2 * 16 * 16, generator=g).sub_(0.5).div_(0.5).pin_memory() for _ in range(BATCH)]
    idss = [ids.clone() for _ in range(BATCH)]
    lib = N.lib()
    lib.rf_launch_count.restype = ctypes.c_uint64

    def prefill():
        eng.prefill_batch(idss, [p.to(dev, non_blocking=True) for p in pxs], [grid] * BATCH)
    prefill()
    c0 = lib.rf_launch_count()
    prefill()
    prefill_launches = int(lib.rf_launch_count() - c0)
    ms, clocks = _timed(prefill, max(3, args.ttft_samples), 3)
    if args.profiler_range:                      # one multimodal prefill for ncu --profile-from-start off
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        prefill()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    prefill()
    c0 = lib.rf_launch_count()
    eng.text.capture(BATCH)
    step_launches = int(lib.rf_launch_count() - c0) // 2        # one eager + one captured step
    eng.decode(max(args.warmup, 3))
    eng.text.reserve_steps(args.steps)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        eng.text.graphs[BATCH].replay()
    e1.record()
    torch.cuda.synchronize()
    dec_ms = e0.elapsed_time(e1) / args.steps
    eng.text.advance_lengths(args.steps)
    eng.text.check_status()
    eng.close()
    return {
        "metric": "qwen3vl_decode_tokens_per_s", "value": BATCH * 1000.0 / dec_ms, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dec_ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "impl": "ours",
        "config": {"model": "qwen3-vl-2b-architecture random-init", "global_batch": BATCH, "images": "2 x 448x448 per sample",
                   "seq_len": int(ids.numel()), "parallelism": "tp1", "l2": "weights (4 GB) exceed L2"},
        "prefill_ms_p50": statistics.median(ms), "clocks": clocks, "startup_s": startup_s,
        "e2e": {"value": statistics.median(ms), "unit": "ms (batch prefill incl. pixel H2D)",
                "h2d_bytes_per_step": sum(p.numel() for p in pxs) * 4, "d2h_bytes_per_step": 4 * BATCH},
        "gpu_launches": args.steps * step_launches, "launches_per_decode_step": step_launches,
        "launches_per_prefill": prefill_launches,
    }


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:          # one line per job, also under torch.distributed.run
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    out = {"decode": run, "pi05": run_pi05, "qwen3vl": run_qwen3vl}[args.workload](args)
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
