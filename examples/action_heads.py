#!/usr/bin/env python3
"""The stand-alone action heads and decoders on random weights: build, run once, print latency.

    python examples/action_heads.py --family navdp            # 16-layer diffusion head, DDPM-20, 4 trajectories
    python examples/action_heads.py --family gr00t            # VL encoder + 32-block DiT, 4 Euler steps
    python examples/action_heads.py --family nextdit          # 12 Lumina blocks, 10 Euler steps, 4 trajectories
    python examples/action_heads.py --family rhinovla         # 18-layer expert behind the 72-D head
    python examples/action_heads.py --family rgbd             # two DINOv2 ViT-S towers + perceiver
    python examples/action_heads.py --family gemma4           # six Gemma4 layers at E4B widths, prefill + greedy decode

``--tiny`` uses the small test geometries.  Real checkpoints go through the builders in ``rpu_backend.adapters``
(``build_navdp``, ``build_gr00t_vla``, ``build_nextdit_runtime``, ``build_rpu_expert``, ``build_rgbd_encoder``,
``Gemma4Adapter``); this script only shows the engines' call shapes."""
from __future__ import annotations

import argparse
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


PROFILE = False
BASELINE = False          # also time the plain PyTorch (fp32, eager) formulation of the same call on the same GPU


def vs_eager(what: str, ms: float, fn) -> str:
    if not BASELINE:
        return what
    _, ref_ms = timed(fn, reps=2)
    return f"{what} [PyTorch eager fp32, same GPU: {ref_ms:.1f} ms per call, {ref_ms / ms:.1f}x]"


def timed(fn, reps: int = 5):
    if PROFILE:                      # three warm-up calls, then one call inside a profiler range (ncu --profile-from-start off)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        out = fn()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return out, float("nan")
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        out = fn()
    torch.cuda.synchronize()
    return out, (time.perf_counter() - t0) / reps * 1e3


def navdp(tiny: bool):
    from rhinoforge_b200.models import navdp as m
    cfg = m.tiny_navdp_config() if tiny else m.NavdpConfig()
    eng = m.NavdpEngine(cfg, m.random_navdp_state_dict(cfg, std=0.03), max_samples=4)
    goal, rgbd = torch.randn(1, 1, cfg.hidden), torch.randn(1, cfg.memory_len - 2, cfg.hidden)
    init = torch.randn(4, cfg.predict_size, cfg.action_dim)
    out, ms = timed(lambda: eng.predict_action(goal, rgbd, init, seed=1))
    what = f"actions {tuple(out.shape)}, {cfg.steps} DDPM steps"
    if BASELINE:
        sd32 = {k: v.float() for k, v in m.random_navdp_state_dict(cfg, std=0.03).items()}
        ref = m.TorchNavdp(cfg, {k: v.cuda() for k, v in sd32.items()}, device="cuda")
        step_noise = torch.randn(cfg.steps, *init.shape)
        what = vs_eager(what, ms, lambda: ref.predict_action(goal.cuda(), rgbd.cuda(), init, step_noise))
    return what, ms


def gr00t(tiny: bool):
    from rhinoforge_b200.models import gr00t as m
    cfg = m.tiny_gr00t_config() if tiny else m.Gr00tConfig(embodiments=2, max_pos=64)
    sd = {k: v.half() for k, v in m.random_gr00t_state_dict(cfg).items()}
    eng = m.Gr00tEngine(cfg, sd.__getitem__, embodiment=1, max_vl=256)
    S = 148
    hidden = torch.randn(S, cfg.vl_dim).cuda()
    im = torch.zeros(S, dtype=torch.bool)
    im[4:4 + 64] = True
    state, noise = torch.randn(cfg.state_dim), torch.randn(cfg.horizon, cfg.action_dim)
    out, ms = timed(lambda: eng.denoise(eng.vl_encode(hidden), state, noise, im))
    return f"actions {tuple(out.shape)}, {cfg.steps} Euler steps over {S} VL tokens", ms


def nextdit(tiny: bool):
    from rhinoforge_b200.models import nextdit as m
    cfg = m.tiny_nextdit_config() if tiny else m.NextDiTConfig()
    eng = m.NextDiTEngine(cfg, m.random_nextdit_state_dict(cfg))
    acts, cond = torch.randn(4, cfg.action_seq, cfg.action_dim), torch.randn(1, min(260, cfg.max_cross), cfg.cond_dim)
    ts, dts = torch.linspace(1.0, 0.1, 10), torch.full((10,), -0.1)
    out, ms = timed(lambda: eng.denoise_actions(acts, ts, dts, cond))
    what = f"actions {tuple(out.shape)}, 10 Euler steps"
    if BASELINE:
        ref = m.TorchNextDiT(cfg, {k: v.float().cuda() for k, v in m.random_nextdit_state_dict(cfg).items()}, device="cuda")
        what = vs_eager(what, ms, lambda: ref.denoise_actions(acts, ts.tolist(), dts.tolist(), cond[0].cuda()))
    return what, ms


def rhinovla(tiny: bool):
    from rhinoforge_b200.models import rhinovla as m
    cfg = m.tiny_rhinovla_config() if tiny else m.RhinoVLAConfig()
    eng = m.RhinoVLAEngine(cfg, m.random_rhinovla_state_dict(cfg, std=0.02), max_prefix=512)
    P = 300 if not tiny else 21
    eng.set_prefix([(torch.randn(cfg.kv_heads, P, cfg.head_dim).cuda().half() * 0.5, torch.randn(cfg.kv_heads, P, cfg.head_dim).cuda().half())
                    for _ in range(cfg.layers)])
    state, noise = torch.randn(cfg.state_dim), torch.randn(cfg.horizon, cfg.action_dim)
    out, ms = timed(lambda: eng.predict(state, noise))
    return f"actions {tuple(out.shape)}, {cfg.num_steps} Euler steps over a {P}-row prefix", ms


def rgbd(tiny: bool):
    from rhinoforge_b200.models import rgbd as m
    cfg = m.tiny_rgbd_config() if tiny else m.RgbdConfig()
    enc = m.RgbdEncoder(cfg, m.random_rgbd_state_dict(cfg))
    S = cfg.image_size
    img, dep = torch.rand(1, cfg.memory_size, S, S, 3), torch.rand(1, cfg.memory_size, S, S, 1)
    out, ms = timed(lambda: enc(img, dep))
    what = f"memory tokens {tuple(out.shape)}"
    if BASELINE:
        ref = m.TorchRgbdEncoder(cfg, {k: v.float().cuda() for k, v in m.random_rgbd_state_dict(cfg).items()}, device="cuda")
        what = vs_eager(what, ms, lambda: ref.forward(img, dep))
    return what, ms


def gemma4(tiny: bool):
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig
    from rhinoforge_b200.models.gemma4 import Gemma4Engine
    wide = {} if tiny else dict(hidden_size=2560, intermediate_size=10240, num_attention_heads=8, num_key_value_heads=2,
                                sliding_window=512, hidden_size_per_layer_input=256)
    c = Gemma4TextConfig(**{**dict(vocab_size=2048, vocab_size_per_layer_input=2048, hidden_size=128, intermediate_size=256,
                                   num_hidden_layers=6, num_attention_heads=2, num_key_value_heads=1, head_dim=256, global_head_dim=512,
                                   sliding_window=16, layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2,
                                   num_kv_shared_layers=2, hidden_size_per_layer_input=32, max_position_embeddings=2048), **wide})
    g = torch.Generator().manual_seed(0)
    shapes = {}

    def get(name):                       # random weights on demand, one shape lookup through a meta model
        if not shapes:
            from transformers.models.gemma4.modeling_gemma4 import Gemma4ForCausalLM
            with torch.device("meta"):
                meta = Gemma4ForCausalLM(c)
            shapes.update({k: tuple(v.shape) for k, v in meta.state_dict().items()})
        shape = shapes[name]
        if len(shape) >= 2:
            return torch.randn(shape, generator=g) * (0.5 if "embed" in name else 0.02)
        return torch.ones(shape)
    eng = Gemma4Engine(c, get, max_seq_len=1024, max_batch=1, max_tokens=1024)
    prompt = torch.randint(1, 2048, (600,), generator=g)
    out, ms = timed(lambda: eng.generate([prompt], 16), reps=2)
    return f"600-token prefill + 16 greedy tokens {tuple(out.shape)}", ms


FAMILIES = dict(navdp=navdp, gr00t=gr00t, nextdit=nextdit, rhinovla=rhinovla, rgbd=rgbd, gemma4=gemma4)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--family", choices=sorted(FAMILIES))
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="run the call once inside cudaProfilerStart/Stop after three warm-up calls (for ncu --profile-from-start off)")
    ap.add_argument("--baseline", action="store_true",
                    help="navdp / nextdit / rgbd: also time the PyTorch fp32 eager formulation of the same call on the same GPU")
    ap.add_argument("--check-config", action="store_true", help="validate the arguments and exit without loading torch or the runtime")
    a = ap.parse_args()
    if a.check_config:
        print("configuration OK")
        return 0
    if a.family is None:
        ap.error("--family is required")
    global torch, PROFILE, BASELINE
    import torch
    PROFILE, BASELINE = a.profile, a.baseline
    if not torch.cuda.is_available():
        print("this example needs a CUDA device")
        return 2
    with torch.no_grad():
        what, ms = FAMILIES[a.family](a.tiny)
    print(f"{a.family}: {what}: {ms:.2f} ms per call")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
