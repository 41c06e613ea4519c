#!/usr/bin/env python
"""Kernel micro-benchmarks with roofline fractions (device-timed, L2 flushed between iterations).

    python bench_kernels.py gemm --m 64 --n 12288 --k 4096 --dual [--packed] [--int8]
    python bench_kernels.py attn_prefill --seqs 4 --len 2048 --heads 32 --kv-heads 8 --hd 128
    python bench_kernels.py attn_decode --seqs 64 --len 1024 --heads 32 --kv-heads 8 --hd 128
    python bench_kernels.py gdn --seqs 1 --len 1024 --hk 16 --hv 32
    python bench_kernels.py suite            # the shapes of one Qwen3-8B decode step and prefill chunk

Every line is JSON: the achieved throughput and its fraction of the measured peaks in
``MEASURED_PEAKS.json`` (copy bandwidth and cuBLAS bf16 throughput measured on this pool; the fallback
values 6.65 TB/s and 1.59 PFLOP/s are used, and labelled, when the file is absent).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent


def peaks() -> dict:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.is_file():
        d = json.loads(f.read_text())
        return {"hbm_gbs": float(d.get("hbm_gbs", 6650.0)), "tflops": float(d.get("bf16_tflops", 1590.0)), "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "src": "fallback"}


_flush = None


def flush_l2() -> None:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")      # 2x the 126 MB L2
    _flush.zero_()


def time_graph_us(make_fn, nbuf: int, reps: int = 24) -> float:
    """Back-to-back in-stream time per launch: ``reps`` launches captured in one CUDA graph, cycling over ``nbuf``
    operand sets (``make_fn(i)`` returns the launch closure of set ``i``) so that no launch finds its weights in L2."""
    fns = [make_fn(i) for i in range(nbuf)]
    for f in fns:
        f()
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for i in range(reps):
            fns[i % nbuf]()
    ts = []
    for _ in range(5):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / reps)
    return statistics.median(ts)


def time_us(fn, iters: int = 20, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts)


def report(name: str, us: float, *, flops: float = 0.0, bytes_: float = 0.0, **extra) -> dict:
    pk = peaks()
    out = {"kernel": name, "us": round(us, 2), **extra}
    if flops:
        out["tflops"] = round(flops / us * 1e-6, 1)
        out[f"frac_of_{pk['src']}_tflops"] = round(flops / us * 1e-6 / pk["tflops"], 3)
    if bytes_:
        out["gbs"] = round(bytes_ / us * 1e-3, 1)
        out[f"frac_of_{pk['src']}_hbm"] = round(bytes_ / us * 1e-3 / pk["hbm_gbs"], 3)
    print(json.dumps(out), flush=True)
    return out


def bench_gemm(m, n, k, *, dual=False, packed=False, int8=False, dtype=torch.float16, profile=False, splits=0):
    """In-stream time of one GEMM: launches are chained in a CUDA graph over enough weight copies to defeat L2."""
    from rhinoforge_b200.ops import kernels as K
    rows = 2 * n if dual else n
    wbytes = rows * k * (1 if int8 else 2)
    nbuf = 1 if profile else max(1, min(12, -(-(300 << 20) // wbytes)))
    x = (torch.randn(m, k, device="cuda") * 0.5).to(dtype)
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    sets = []
    for _ in range(nbuf):
        if int8:
            w = torch.randint(-127, 128, (rows, k), device="cuda", dtype=torch.int8)
            sc = (torch.rand(rows, device="cuda") * 0.004 + 0.001).to(dtype)
        else:
            w, sc = (torch.randn(rows, k, device="cuda") * 0.05).to(dtype), None
        sets.append((K.pack_weight(w, 2 if dual else 1) if packed else w, sc))

    def make(i):
        w, sc = sets[i]
        kw = dict(out=out, scale=sc, act="silu_mul" if dual else None, dual=dual, force_splits=splits)
        if packed:
            return lambda: K.gemm(x, w, packed_shape=(rows, k), **kw)
        return lambda: K.gemm(x, w, **kw)
    if profile:
        fn = make(0)
        fn(); torch.cuda.synchronize()
        torch.cuda.profiler.start(); fn(); torch.cuda.synchronize(); torch.cuda.profiler.stop()
        return None
    us = time_graph_us(make, nbuf)
    return report("gemm", us, flops=2.0 * m * rows * k, bytes_=wbytes + m * k * 2 + m * n * 2, m=m, n=n, k=k, dual=dual,
                  packed=packed, int8=int8, splits=splits or "auto", plan=_plan(m, n, k, dual, packed, int8, dtype, splits))


def _plan(m, n, k, dual, packed, int8, dtype, splits):
    """The launch plan the library picks for this shape (swap-AB, tile width, splits, stages, grid, shared memory)."""
    from rhinoforge_b200.ops.kernels import gemm_plan
    try:
        return gemm_plan(m, n, k, dtype=dtype, dual=dual, packed=packed, int8=int8, force_splits=splits)
    except Exception:  # noqa: BLE001  (diagnostic only)
        return None


def bench_attn_prefill(seqs, length, heads, kv_heads, hd, *, causal=True, dtype=torch.float16, profile=False):
    from rhinoforge_b200.ops import kernels as K
    T = seqs * length
    qkv = (torch.randn(T, (heads + 2 * kv_heads) * hd, device="cuda") * 0.5).to(dtype)
    out = torch.empty(T, heads * hd, dtype=dtype, device="cuda")
    ql = torch.full((seqs,), length, dtype=torch.int32, device="cuda")
    qs = (torch.arange(seqs, dtype=torch.int32, device="cuda") * length).contiguous()
    q, k, v = qkv[:, :heads * hd], qkv[:, heads * hd:(heads + kv_heads) * hd], qkv[:, (heads + kv_heads) * hd:]
    fn = lambda: K.attention_prefill(q, out, Hq=heads, Hkv=kv_heads, hd=hd, q_start=qs, q_len=ql, kv_len=ql, max_q_len=length,
                                     k=k, v=v, kv_start=qs, causal=causal)
    if profile:
        fn(); torch.cuda.synchronize()
        torch.cuda.profiler.start(); fn(); torch.cuda.synchronize(); torch.cuda.profiler.stop()
        return None
    us = time_us(fn)
    flops = 4.0 * seqs * heads * length * length * hd * (0.5 if causal else 1.0)
    return report("attn_prefill", us, flops=flops, seqs=seqs, len=length, heads=heads, kv_heads=kv_heads, hd=hd, causal=causal)


def bench_attn_decode(seqs, length, heads, kv_heads, hd, *, dtype=torch.float16):
    from rhinoforge_b200.ops import kernels as K
    from rhinoforge_b200.runtime.kv_cache import PagedKV
    cache = PagedKV(1, seqs, length + 16, kv_heads, hd, dtype=dtype)
    cache.reserve_all()
    cache.kv.normal_(0, 0.5)
    q = (torch.randn(seqs, heads * hd, device="cuda") * 0.5).to(dtype)
    out = torch.empty_like(q)
    kl = torch.full((seqs,), length, dtype=torch.int32, device="cuda")
    ws = K.attn_decode_scratch(seqs, heads, hd, q.device)
    fn = lambda: K.attention_decode(q, out, Hq=heads, Hkv=kv_heads, hd=hd, kv_len=kl, max_kv_len=length, k_pool=cache.kv[0, 0],
                                    v_pool=cache.kv[0, 1], page_table=cache.page_table, ws=ws)
    us = time_us(fn)
    r = report("attn_decode", us, bytes_=2.0 * seqs * length * kv_heads * hd * 2, seqs=seqs, len=length, heads=heads,
               kv_heads=kv_heads, hd=hd)
    cache.close()
    return r


def bench_gdn(seqs, length, hk, hv, *, dk=128, dv=128, dtype=torch.float16):
    from rhinoforge_b200.ops import kernels as K
    T = seqs * length
    qkv = torch.randn(T, 2 * hk * dk + hv * dv, device="cuda").to(dtype)
    ba = torch.randn(T, 2 * ((hv + 7) // 8 * 8), device="cuda").to(dtype)
    half = ba.shape[1] // 2
    state = torch.zeros(seqs, hv, dk, dv, device="cuda")
    A, dtb = torch.zeros(hv, device="cuda"), torch.zeros(hv, device="cuda")
    ql = torch.full((seqs,), length, dtype=torch.int32, device="cuda")
    qs = (torch.arange(seqs, dtype=torch.int32, device="cuda") * length).contiguous()
    if length == 1:
        fn = lambda: K.gdn_recurrent(qkv, ba[:, :half], ba[:, half:], state, A, dtb, Hk=hk, Hv=hv, Dk=dk, Dv=dv)
    else:
        fn = lambda: K.gdn_recurrent(qkv, ba[:, :half], ba[:, half:], state, A, dtb, Hk=hk, Hv=hv, Dk=dk, Dv=dv, q_start=qs, q_len=ql)
    us = time_us(fn, iters=10)
    return report("gdn_recurrent", us, flops=6.0 * T * hv * dk * dv, bytes_=2.0 * seqs * hv * dk * dv * 4, seqs=seqs, len=length,
                  hk=hk, hv=hv, us_per_token=round(us / length, 3))


def time_hot_us(fn, n: int = 50) -> float:
    """Mean in-stream time of ``n`` back-to-back launches of one closure in a CUDA graph, operands L2-resident: the regime
    of the action heads' denoise loops, where the same few MB of weights serve every step."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for _ in range(n):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (5 * n)


def heads() -> None:
    """The latency-bound shapes of the action heads: short attention with and without the host-side key bound (which
    selects the register-accumulator kernel), and few-row GEMMs on the kernel the router picks (set ``RF_GEMM_SMALL=0`` to
    time the streaming kernel on the same shapes) against ``torch.matmul``."""
    import math
    from rhinoforge_b200.ops import kernels as K
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    for name, B, Q, KV, H, hd in (("navdp self", 4, 24, 24, 8, 64), ("navdp cross", 4, 24, 34, 8, 64), ("nextdit self", 4, 32, 32, 12, 64),
                                  ("nextdit cross", 4, 32, 260, 12, 64), ("gr00t self", 1, 41, 41, 32, 64), ("gr00t cross", 1, 41, 148, 32, 64),
                                  ("rgbd self", 1, 32, 32, 6, 64), ("50x350 hd128", 1, 50, 350, 16, 128), ("64x512 hd128", 2, 64, 512, 16, 128)):
        q = torch.randn(B * Q, H * hd, device="cuda", dtype=torch.float16) * 0.3
        k = torch.randn(B * KV, H * hd, device="cuda", dtype=torch.float16) * 0.3
        v = torch.randn(B * KV, H * hd, device="cuda", dtype=torch.float16)
        out = torch.empty_like(q)
        qs, ql, ks, kl = i32([j * Q for j in range(B)]), i32([Q] * B), i32([j * KV for j in range(B)]), i32([KV] * B)
        r = {}
        for arm, bound in (("bounded_us", KV), ("unbounded_us", 0)):
            r[arm] = round(time_hot_us(lambda: K.attention_prefill(q, out, Hq=H, Hkv=H, hd=hd, q_start=qs, q_len=ql, kv_len=kl, max_q_len=Q,
                                                                   k=k, v=v, kv_start=ks, causal=False, scale=1 / math.sqrt(hd),
                                                                   max_kv_len=bound)), 2)
        print(json.dumps({"kernel": "attention_prefill", "case": name, "seqs": B, "q": Q, "kv": KV, "heads": H, "hd": hd, **r}), flush=True)
    for M, N, Kd, dual in ((128, 384, 1536, False), (128, 1536, 384, False), (128, 1152, 384, False), (96, 384, 384, False), (24, 1152, 384, False),
                           (24, 384, 384, False), (31, 1024, 1024, False), (31, 2560, 1024, False), (31, 4096, 1024, True), (50, 2560, 1024, False),
                           (50, 4096, 1024, True), (50, 1024, 2048, False), (41, 4608, 1536, False), (41, 1536, 6144, False)):
        x = torch.randn(M, Kd, device="cuda", dtype=torch.float16)
        w = torch.randn(N * (2 if dual else 1), Kd, device="cuda", dtype=torch.float16) * 0.05
        wp = K.pack_weight(w, sections=2) if dual else K.pack_weight(w)
        out = torch.empty(M, N, device="cuda", dtype=torch.float16)
        kw = dict(act="silu_mul", dual=True) if dual else {}
        us = time_hot_us(lambda: K.gemm(x, wp, packed_shape=(w.shape[0], Kd), out=out, **kw))
        ref = torch.empty(M, w.shape[0], device="cuda", dtype=torch.float16)
        lib = time_hot_us(lambda: torch.matmul(x, w.t(), out=ref))
        print(json.dumps({"kernel": "gemm", "m": M, "n": N, "k": Kd, "dual": dual, "small_kernel": os.environ.get("RF_GEMM_SMALL", "1") != "0",
                          "us": round(us, 2), "torch_matmul_us": round(lib, 2)}), flush=True)


def sweep() -> None:
    """Split-K factors around the planner's choice for the Qwen3-8B decode GEMMs and two mid-size GEMMs."""
    for shape in ((64, 6144, 4096, False), (64, 4096, 4096, False), (64, 12288, 4096, True), (64, 4096, 12288, False),
                  (1, 4096, 4096, False), (768, 6144, 1152, False), (768, 1152, 4304, False), (968, 2048, 16384, False)):
        m, n, k, dual = shape
        for sp in (0, 1, 2, 3, 4, 6, 8):
            if sp > max(1, (k // 64) // 4):
                continue
            bench_gemm(m, n, k, dual=dual, packed=True, splits=sp)


def suite() -> None:
    """Qwen3-8B shapes: the four decode GEMMs at 64 tokens, the same at 2048 tokens, attention at both."""
    for packed in (True,):
        for m in (64, 2048):
            bench_gemm(m, 6144, 4096, packed=packed)                 # qkv
            bench_gemm(m, 4096, 4096, packed=packed)                 # o_proj
            bench_gemm(m, 12288, 4096, dual=True, packed=packed)     # gate/up + SwiGLU
            bench_gemm(m, 4096, 12288, packed=packed)                # down
    bench_gemm(64, 151936, 4096, packed=True)                        # lm_head
    bench_gemm(64, 12288, 4096, dual=True, packed=True, int8=True)
    bench_attn_decode(64, 1024, 32, 8, 128)
    bench_attn_prefill(4, 2048, 32, 8, 128)
    bench_attn_prefill(1, 968, 8, 1, 256, causal=False)              # Pi0.5 prefix
    bench_attn_prefill(3, 256, 16, 16, 128, causal=False)            # SigLIP (72 padded to 128)
    bench_gdn(1, 1, 16, 32)
    bench_gdn(1, 1024, 16, 32)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["gemm", "attn_prefill", "attn_decode", "gdn", "suite", "sweep", "heads"])
    for name, d in (("m", 64), ("n", 4096), ("k", 4096), ("seqs", 4), ("len", 2048), ("heads", 32), ("kv-heads", 8),
                    ("hd", 128), ("hk", 16), ("hv", 32)):
        ap.add_argument(f"--{name}", type=int, default=d)
    ap.add_argument("--splits", type=int, default=0, help="force the split-K factor (0: planner)")
    ap.add_argument("--dual", action="store_true")
    ap.add_argument("--packed", action="store_true")
    ap.add_argument("--int8", action="store_true")
    ap.add_argument("--bidirectional", action="store_true")
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="run the kernel once inside cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    a = ap.parse_args()
    dt = torch.bfloat16 if a.bf16 else torch.float16
    if a.what == "gemm":
        bench_gemm(a.m, a.n, a.k, dual=a.dual, packed=a.packed, int8=a.int8, dtype=dt, profile=a.profile, splits=a.splits)
    elif a.what == "attn_prefill":
        bench_attn_prefill(a.seqs, a.len, a.heads, a.kv_heads, a.hd, causal=not a.bidirectional, dtype=dt, profile=a.profile)
    elif a.what == "attn_decode":
        bench_attn_decode(a.seqs, a.len, a.heads, a.kv_heads, a.hd, dtype=dt)
    elif a.what == "gdn":
        bench_gdn(a.seqs, a.len, a.hk, a.hv, dtype=dt)
    elif a.what == "sweep":
        sweep()
    elif a.what == "heads":
        heads()
    else:
        suite()
    return 0


if __name__ == "__main__":
    sys.exit(main())
