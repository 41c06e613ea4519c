"""NavDP host-side pieces: DDPM tables, memory rows, the fp32 oracle's structure, checkpoint validation."""
import math

import pytest
import torch

from rhinoforge_b200.models import navdp as nd


def test_ddpm_tables_invariants():
    ts, coeff, sigma = nd.ddpm_tables(20)
    assert ts == list(range(19, -1, -1))
    assert coeff.shape == (20, 4) and sigma.shape == (20,)
    # last step: the clean-sample estimate passes through unchanged and no noise is added
    assert abs(float(coeff[-1, 2]) - 1.0) < 1e-6 and abs(float(coeff[-1, 3])) < 1e-7 and float(sigma[-1]) == 0.0
    assert (sigma[:-1] > 0).all()
    # x0 = A x + B eps inverts x = sqrt(ap) x0 + sqrt(1 - ap) eps
    A, B = coeff[:, 0].double(), coeff[:, 1].double()
    ap = 1.0 / A ** 2
    assert torch.allclose(-B / A, (1 - ap).sqrt(), atol=1e-5)
    assert (ap[1:] > ap[:-1]).all() and float(ap[0]) < 0.01 and float(ap[-1]) > 0.98


def test_ddpm_step_is_posterior_mean():
    steps = 20
    ts, coeff, _ = nd.ddpm_tables(steps)
    bar = lambda u: math.cos((u + 0.008) / 1.008 * math.pi / 2) ** 2
    betas = [min(1 - bar((i + 1) / steps) / bar(i / steps), 0.999) for i in range(steps)]
    ac = torch.cumprod(1 - torch.tensor(betas, dtype=torch.float64), 0)
    k = 7
    t = ts[k]
    x, x0 = 0.3, -0.4
    beta_t = 1 - float(ac[t] / ac[t - 1])
    mean = (float(ac[t - 1]) ** 0.5 * beta_t * x0 + (1 - beta_t) ** 0.5 * (1 - float(ac[t - 1])) * x) / (1 - float(ac[t]))
    assert abs(float(coeff[k, 2]) * x0 + float(coeff[k, 3]) * x - mean) < 1e-6


def test_memory_rows_layout():
    cfg = nd.tiny_navdp_config()
    sd = nd.random_navdp_state_dict(cfg)
    ts, _, _ = nd.ddpm_tables(cfg.steps)
    goal, rgbd = torch.randn(1, 1, cfg.hidden), torch.randn(1, cfg.memory_len - 2, cfg.hidden)
    mem = nd.memory_rows(sd, cfg, ts, goal, rgbd)
    assert mem.shape == (cfg.steps, cfg.memory_len, cfg.hidden)
    pos = sd["cond_pos_embed"][0]
    assert torch.allclose(mem[3, 1] - pos[1], goal[0, 0], atol=1e-6)
    assert torch.allclose(mem[0, 2:] - pos[2:], rgbd[0], atol=1e-6)
    te = nd.sinusoidal_time_embedding(torch.tensor([float(ts[2])]), cfg.hidden)[0]
    assert torch.allclose(mem[2, 0] - pos[0], te, atol=1e-6)
    with pytest.raises(ValueError, match="memory has"):
        nd.memory_rows(sd, cfg, ts, goal, rgbd[:, :-1])


def test_oracle_is_causal_over_action_tokens_and_deterministic():
    cfg = nd.tiny_navdp_config()
    sd = nd.random_navdp_state_dict(cfg, seed=3)
    o = nd.TorchNavdp(cfg, sd)
    mem = torch.randn(1, cfg.memory_len, cfg.hidden)
    x = torch.randn(2, cfg.predict_size, cfg.action_dim)
    e0 = o.predict_noise(x, mem)
    x2 = x.clone()
    x2[:, 5:] += 1.0
    e1 = o.predict_noise(x2, mem)
    assert torch.allclose(e0[:, :5], e1[:, :5], atol=1e-5) and not torch.allclose(e0[:, 5:], e1[:, 5:], atol=1e-3)
    g = torch.Generator().manual_seed(0)
    init = torch.randn(2, cfg.predict_size, cfg.action_dim, generator=g)
    zs = torch.randn(cfg.steps, 2, cfg.predict_size, cfg.action_dim, generator=g)
    goal, rgbd = torch.randn(1, 1, cfg.hidden, generator=g), torch.randn(1, cfg.memory_len - 2, cfg.hidden, generator=g)
    a, b = o.predict_action(goal, rgbd, init, zs), o.predict_action(goal, rgbd, init, zs)
    assert torch.equal(a, b) and a.shape == init.shape and float(a.abs().max()) <= 1.0 + 1e-5


def test_check_state_dict_names_the_mismatch():
    cfg = nd.tiny_navdp_config()
    sd = nd.random_navdp_state_dict(cfg)
    nd.check_state_dict(cfg, sd)
    del sd["decoder.layers.1.norm3.bias"]
    sd["action_head.weight"] = torch.zeros(4, cfg.hidden)
    with pytest.raises(ValueError, match="norm3.bias: missing") as e:
        nd.check_state_dict(cfg, sd)
    assert "action_head.weight: (4, 96) float32, expected (3, 96)" in str(e.value)


def test_full_profile_parameter_count():
    cfg = nd.NavdpConfig()
    n = sum(math.prod(s) for _, s, _ in nd.navdp_shapes(cfg))
    per_layer = 2 * (3 * 384 * 384 + 3 * 384 + 384 * 384 + 384) + 2 * 384 * 1536 + 1536 + 384 + 6 * 384
    assert n == 16 * per_layer + (384 * 3 + 384) + 32 * 384 + 34 * 384 + 2 * 384 + 3 * 384 + 3


def test_adapter_manifest_and_profile_checks(tmp_path):
    from safetensors.torch import save_file
    from rhinoforge_b200.adapters import navdp as ad
    from rhinoforge_b200.adapters._assets import sha256_of
    cfg = nd.tiny_navdp_config()
    path = tmp_path / "navdp_head.safetensors"
    save_file(nd.random_navdp_state_dict(cfg), str(path))
    with pytest.raises(ValueError, match="does not match the manifest"):
        ad.load_navdp_tensors(path, asset_manifest={str(path): "0" * 64})
    with pytest.raises(ValueError, match="not listed"):
        ad.load_navdp_tensors(path, asset_manifest={"other.safetensors": "0" * 64})
    sd = ad.load_navdp_tensors(path, asset_manifest={"navdp_head.safetensors": sha256_of(path)})
    assert set(sd) == {n for n, _, _ in nd.navdp_shapes(cfg)}
    with pytest.raises(ValueError, match=r"decoder layers \[0, 1\]; the profile is 0..15"):
        ad.build_navdp(path, device="cpu")


def test_runtime_draws_noise_from_the_seed_and_validates_timesteps():
    from rhinoforge_b200.adapters.navdp import NavdpRuntime
    cfg = nd.tiny_navdp_config()
    calls = {}

    class FakeEngine:
        def __init__(self):
            self.cfg = cfg

        def predict_action(self, goal, rgbd, init, zs):
            calls["init"], calls["zs"] = init, zs
            return init + zs.sum(0)

        def predict_noise(self, x, k, goal, rgbd):
            calls["k"] = k
            return x

        def check_status(self):
            calls["checked"] = True

        def close(self):
            calls["closed"] = True

    rt = NavdpRuntime(FakeEngine())
    a = rt.predict_action(None, None, sample_num=3, seed=11)
    b = rt.predict_action(None, None, sample_num=3, seed=11)
    assert torch.equal(a, b) and a.shape == (3, cfg.predict_size, cfg.action_dim) and calls["checked"]
    assert calls["zs"].shape == (cfg.steps, 3, cfg.predict_size, cfg.action_dim)
    assert not torch.equal(a, rt.predict_action(None, None, sample_num=3, seed=12))
    rt.predict_noise(torch.zeros(1, cfg.predict_size, cfg.action_dim), torch.tensor([cfg.steps - 1]), None, None)
    assert calls["k"] == 0
    with pytest.raises(ValueError, match="outside"):
        rt.predict_noise(torch.zeros(1, cfg.predict_size, cfg.action_dim), cfg.steps, None, None)
    rt.destroy()
    assert calls["closed"]
