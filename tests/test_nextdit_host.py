"""InternVLA-N1 NextDiT, host side: profile, oracle structure, adapter flattening and checks."""
import pytest
import torch

from rhinoforge_b200.models import nextdit as nx


def test_profile_shapes_and_time_frequencies():
    cfg = nx.NextDiTConfig()
    shapes = {n: s for n, s, _ in nx.nextdit_shapes(cfg)}
    assert shapes["model.layers.11.norm1.linear.weight"] == (1536, 384)
    assert shapes["model.layers.0.gate"] == (6,)
    assert shapes["model.norm_out.linear_1.weight"] == (384, 384)
    f = nx.time_frequencies(torch.tensor([0.0, 2.0]), 8)
    assert torch.allclose(f[0], torch.tensor([1.0] * 4 + [0.0] * 4))
    assert abs(float(f[1, 0]) - torch.cos(torch.tensor(2.0)).item()) < 1e-6 and abs(float(f[1, 4]) - torch.sin(torch.tensor(2.0)).item()) < 1e-6


def test_oracle_trajectories_are_independent_and_condition_matters():
    cfg = nx.tiny_nextdit_config()
    sd = nx.random_nextdit_state_dict(cfg, seed=1)
    o = nx.TorchNextDiT(cfg, sd)
    g = torch.Generator().manual_seed(0)
    acts = torch.randn(2, cfg.action_seq, cfg.action_dim, generator=g)
    cond = torch.randn(9, cfg.cond_dim, generator=g)
    ts, dts = [1.0, 0.6, 0.2], [-0.4, -0.4, -0.2]
    out = o.denoise_actions(acts, ts, dts, cond)
    assert out.shape == acts.shape
    assert torch.allclose(out[1], o.denoise_actions(acts[1:], ts, dts, cond)[0], atol=1e-6)
    assert not torch.allclose(out, o.denoise_actions(acts, ts, dts, cond + 0.5), atol=1e-4)
    # a zero cross gate removes the cross branch, not the caption's effect on the modulation
    sd0 = dict(sd)
    for i in range(cfg.layers):
        sd0[f"model.layers.{i}.gate"] = torch.zeros(cfg.heads)
    o0 = nx.TorchNextDiT(cfg, sd0)
    a, b = o0.velocity(acts[0], 0.5, cond), o0.velocity(acts[0], 0.5, cond.flip(0))
    assert torch.allclose(a, b, atol=1e-5)                    # only the pooled mean of the caption is left


def test_adapter_flattens_modules_and_checks_geometry():
    from rhinoforge_b200.adapters.internvla_n1 import nextdit as ad
    from rhinoforge_b200.api.errors import UnsupportedModelError
    cfg = nx.tiny_nextdit_config()
    sd = nx.random_nextdit_state_dict(cfg, seed=2)
    inner = {k[len("model."):]: v for k, v in sd.items() if k.startswith("model.")}
    enc, dec = torch.nn.Linear(cfg.action_dim, cfg.hidden), torch.nn.Linear(cfg.hidden, cfg.action_dim)
    flat = ad.nextdit_state_dict(inner, enc, dec, sd["action_position"][None])
    assert set(flat) == set(sd) and flat["action_position"].shape == (cfg.action_seq, cfg.hidden)
    got = ad.config_from(flat, heads=cfg.heads, max_cross_seq_len=cfg.max_cross)
    assert got == cfg
    with pytest.raises(UnsupportedModelError, match="geometry"):
        ad.preflight(got)
    ad.preflight(got, strict=False)
    with pytest.raises(TypeError, match="missing"):
        ad.nextdit_state_dict(torch.nn.Linear(2, 2))
    with pytest.raises(ValueError, match="needs `action_encoder`"):
        ad.build_nextdit_runtime(inner, device="cpu")


def test_runtime_shape_checks_and_forward_actions():
    from rhinoforge_b200.adapters.internvla_n1.nextdit import NextDiTRuntime
    cfg = nx.tiny_nextdit_config()

    class Fake:
        def __init__(self):
            self.cfg = cfg

        def denoise_actions(self, a, ts, dts, cond, reuse_condition=True):
            return a.float() + float(dts.sum()) * 2.0

        def check_status(self):
            pass

        def close(self):
            self.closed = True

    rt = NextDiTRuntime(Fake())
    a = torch.zeros(2, cfg.action_seq, cfg.action_dim)
    cond = torch.zeros(1, 5, cfg.cond_dim)
    assert torch.allclose(rt.forward_actions(a, torch.tensor(0.3), cond), torch.full_like(a, 2.0))
    with pytest.raises(ValueError, match="actions must be"):
        rt.denoise_actions(torch.zeros(5, cfg.action_seq, cfg.action_dim), torch.ones(1), torch.ones(1), cond)
    with pytest.raises(ValueError, match="condition must be"):
        rt.denoise_actions(a, torch.ones(1), torch.ones(1), torch.zeros(2, 5, cfg.cond_dim))
    rt.destroy()
    assert rt.engine.closed
