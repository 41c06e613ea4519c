"""InternVLA-N1 NextDiT on the accelerator against the fp32 oracle."""
import pytest
import torch

from rhinoforge_b200.models import nextdit as nx

pytestmark = pytest.mark.gpu


def _case(cfg, b, S, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(b, cfg.action_seq, cfg.action_dim, generator=g), torch.randn(1, S, cfg.cond_dim, generator=g)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_single_velocity_matches_oracle(dtype):
    cfg = nx.tiny_nextdit_config()
    sd = nx.random_nextdit_state_dict(cfg, seed=1)
    acts, cond = _case(cfg, 1, 11)
    want = nx.TorchNextDiT(cfg, sd).velocity(acts[0], 0.7, cond[0])
    eng = nx.NextDiTEngine(cfg, sd, dtype=dtype)
    got = eng.denoise_actions(acts, torch.tensor([0.7]), torch.tensor([1.0]), cond, use_graph=False).cpu()[0] - acts[0]
    eng.check_status()
    tol = 3e-2 if dtype == torch.float16 else 1.5e-1
    assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max()))


def test_schedule_batch_and_condition_changes_share_graphs():
    cfg = nx.tiny_nextdit_config()
    sd = nx.random_nextdit_state_dict(cfg, seed=2)
    oracle = nx.TorchNextDiT(cfg, sd)
    eng = nx.NextDiTEngine(cfg, sd)
    ts, dts = torch.tensor([1.0, 0.75, 0.5, 0.25]), torch.tensor([-0.25] * 4)
    acts, cond = _case(cfg, 3, 17)
    want = oracle.denoise_actions(acts, ts.tolist(), dts.tolist(), cond[0])
    got = eng.denoise_actions(acts, ts, dts, cond).cpu()
    assert float((got - want).abs().max()) < 4e-2 * max(1.0, float(want.abs().max()))
    assert torch.equal(got, eng.denoise_actions(acts, ts, dts, cond).cpu())
    assert torch.equal(got, eng.denoise_actions(acts, ts, dts, cond, use_graph=False).cpu())
    # another condition length and another schedule of the same length replay the same graph
    acts2, cond2 = _case(cfg, 3, 6, seed=3)
    ts2, dts2 = torch.tensor([0.9, 0.5, 0.3, 0.1]), torch.tensor([-0.4, -0.2, -0.2, -0.1])
    want2 = oracle.denoise_actions(acts2, ts2.tolist(), dts2.tolist(), cond2[0])
    got2 = eng.denoise_actions(acts2, ts2, dts2, cond2).cpu()
    assert len(eng._graphs) == 1
    assert float((got2 - want2).abs().max()) < 4e-2 * max(1.0, float(want2.abs().max()))
    eng.check_status()


def test_full_profile():
    cfg = nx.NextDiTConfig()
    sd = nx.random_nextdit_state_dict(cfg, seed=4)
    oracle = nx.TorchNextDiT(cfg, sd, device="cuda")
    eng = nx.NextDiTEngine(cfg, sd)
    acts, cond = _case(cfg, 4, 260, seed=5)
    ts, dts = torch.linspace(1.0, 0.1, 10), torch.full((10,), -0.1)
    want = oracle.denoise_actions(acts, ts.tolist(), dts.tolist(), cond[0]).cpu()
    got = eng.denoise_actions(acts, ts, dts, cond).cpu()
    eng.check_status()
    assert torch.isfinite(got).all()
    assert float((got - want).abs().max()) < 5e-2 * max(1.0, float(want.abs().max()))
