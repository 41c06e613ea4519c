"""NavDP on the accelerator against the fp32 ``torch.nn.TransformerDecoder`` oracle."""
import pytest
import torch

from rhinoforge_b200.models import navdp as nd

pytestmark = pytest.mark.gpu


def _inputs(cfg, b, seed=0):
    g = torch.Generator().manual_seed(seed)
    init = torch.randn(b, cfg.predict_size, cfg.action_dim, generator=g)
    zs = torch.randn(cfg.steps, b, cfg.predict_size, cfg.action_dim, generator=g)
    goal = torch.randn(1, 1, cfg.hidden, generator=g)
    rgbd = torch.randn(1, cfg.memory_len - 2, cfg.hidden, generator=g)
    return goal, rgbd, init, zs


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_single_step_noise_matches_oracle(dtype):
    cfg = nd.tiny_navdp_config(steps=1)
    sd = nd.random_navdp_state_dict(cfg, seed=1)
    goal, rgbd, init, zs = _inputs(cfg, 3)
    oracle = nd.TorchNavdp(cfg, sd)
    ts, coeff, _ = nd.ddpm_tables(1)
    mem = nd.memory_rows(oracle.sd, cfg, ts, goal, rgbd)
    eps = oracle.predict_noise(init, mem[0:1])
    eng = nd.NavdpEngine(cfg, sd, max_samples=4, dtype=dtype)
    eng.predict_action(goal, rgbd, init, zs, use_graph=False)
    eng.check_status()
    got = eng.eps[:3 * cfg.predict_size, :cfg.action_dim].float().cpu().reshape(eps.shape)
    tol = 2e-2 if dtype == torch.float16 else 8e-2
    assert float((got - eps).abs().max()) < tol * max(1.0, float(eps.abs().max()))


def test_ddpm_loop_matches_oracle_and_graph_replays():
    cfg = nd.tiny_navdp_config()
    sd = nd.random_navdp_state_dict(cfg, seed=2)
    goal, rgbd, init, zs = _inputs(cfg, 2, seed=5)
    want = nd.TorchNavdp(cfg, sd).predict_action(goal, rgbd, init, zs)
    eng = nd.NavdpEngine(cfg, sd, max_samples=2)
    eager = eng.predict_action(goal, rgbd, init, zs, use_graph=False).cpu()
    g1 = eng.predict_action(goal, rgbd, init, zs).cpu()
    g2 = eng.predict_action(goal, rgbd, init, zs).cpu()
    eng.check_status()
    assert torch.equal(g1, g2) and torch.equal(eager, g1)
    assert float((g1 - want).abs().max()) < 5e-2
    # a second batch size builds its own graph and leaves the first intact
    one = eng.predict_action(goal, rgbd, init[:1], zs[:, :1]).cpu()
    assert float((one - want[:1]).abs().max()) < 5e-2
    assert torch.equal(eng.predict_action(goal, rgbd, init, zs).cpu(), g1)


def test_full_profile_runs_and_stays_in_range():
    cfg = nd.NavdpConfig()
    sd = nd.random_navdp_state_dict(cfg, seed=4, std=0.03)
    goal, rgbd, init, zs = _inputs(cfg, 2, seed=7)
    want = nd.TorchNavdp(cfg, sd, device="cuda").predict_action(goal, rgbd, init, zs).cpu()
    eng = nd.NavdpEngine(cfg, sd, max_samples=2)
    got = eng.predict_action(goal, rgbd, init, zs).cpu()
    eng.check_status()
    assert torch.isfinite(got).all() and float(got.abs().max()) <= 1.0 + 1e-3
    assert float((got - want).abs().mean()) < 3e-2


def test_navdp_through_the_op_surface():
    import json
    import rhinoforge_b200.ops.torch_ops  # noqa: F401  (registers torch.ops.rpu)
    ops = torch.ops.rpu
    cfg = nd.tiny_navdp_config()
    sd = nd.random_navdp_state_dict(cfg, seed=2)
    goal, rgbd, init, zs = _inputs(cfg, 2, seed=5)
    want = nd.TorchNavdp(cfg, sd).predict_action(goal, rgbd, init, zs)
    h = ops.navdp_create(json.dumps({**cfg.__dict__, "rpu_max_samples": 2}))
    ops.navdp_set_weights(h, list(sd), [sd[k] for k in sd])
    got = ops.navdp_forward(h, goal, rgbd, init, zs).cpu()
    assert float((got - want).abs().max()) < 5e-2
    ops.navdp_destroy(h)
    with pytest.raises(Exception, match="unknown or destroyed"):
        ops.navdp_forward(h, goal, rgbd, init, zs)
