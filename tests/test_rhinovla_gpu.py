"""RhinoVLA expert on the accelerator against the fp32 oracle."""
import pytest
import torch

from rhinoforge_b200.models import rhinovla as r

pytestmark = pytest.mark.gpu


def _case(cfg, P, seed=0):
    g = torch.Generator().manual_seed(seed)
    kv = [(torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g) * 0.5, torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g))
          for _ in range(cfg.layers)]
    state, noise = torch.randn(cfg.state_dim, generator=g), torch.randn(cfg.horizon, cfg.action_dim, generator=g)
    am = torch.ones(cfg.horizon, cfg.action_dim)
    am[:, -2:] = 0
    sm = torch.ones(cfg.state_dim)
    sm[-1] = 0
    return kv, state, sm, noise, am


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_denoise_matches_oracle(dtype):
    cfg = r.tiny_rhinovla_config()
    sd = r.random_rhinovla_state_dict(cfg, dtype=torch.float32, seed=1)
    kv, state, sm, noise, am = _case(cfg, 21)
    valid = torch.ones(21, dtype=torch.bool)
    valid[-3:] = False                                         # right padding of the prefix
    cond = r.default_cond_table(cfg, cfg.num_steps)
    want = r.TorchRhinoVLA(cfg, sd).sample_actions(kv, valid, state, sm, noise, am, cond)
    eng = r.RhinoVLAEngine(cfg, sd, max_prefix=64, dtype=dtype)
    eng.set_prefix([(k.cuda().to(dtype), v.cuda().to(dtype)) for k, v in kv], valid)
    got = eng.predict(state, noise, state_mask=sm, action_mask=am).float().cpu()
    eng.check_status()
    tol = 3e-2 if dtype == torch.float16 else 1.5e-1
    assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max()))
    assert float(got[:, -2:].abs().max()) == 0.0
    again = eng.predict(state, noise, state_mask=sm, action_mask=am).float().cpu()
    eager = eng.predict(state, noise, state_mask=sm, action_mask=am, use_graph=False).float().cpu()
    assert torch.equal(got, again) and torch.equal(got, eager)


def test_adapter_with_lora_and_full_profile():
    from rhinoforge_b200.adapters.rhinovla import build_rpu_expert
    cfg = r.RhinoVLAConfig(width=1024, layers=4, heads=16, kv_heads=8, head_dim=128, inter=2048)
    sd = r.random_rhinovla_state_dict(cfg, dtype=torch.float32, seed=3, std=0.02)
    g = torch.Generator().manual_seed(4)
    name = "expert.layers.1.self_attn.q_proj"
    lora = {name + ".lora_A.weight": torch.randn(8, cfg.width, generator=g) * 0.05,
            name + ".lora_B.weight": torch.randn(cfg.heads * cfg.head_dim, 8, generator=g) * 0.05}
    merged = r.merge_lora(sd, lora, scale=2.0)
    kv, state, sm, noise, am = _case(cfg, 100, seed=5)
    valid = torch.ones(100, dtype=torch.bool)
    want = r.TorchRhinoVLA(cfg, merged, device="cuda").sample_actions(kv, valid, state, sm, noise, am, r.default_cond_table(cfg, 10)).cpu()
    expert = {k[len("expert."):]: v for k, v in sd.items() if k.startswith("expert.")}
    io = {k[len("io."):]: v for k, v in sd.items() if k.startswith("io.")}
    eng = build_rpu_expert(expert, action_io=io, mask_proj=None, heads=cfg.heads, kv_heads=cfg.kv_heads, horizon=cfg.horizon,
                           max_seq_len=256, lora=lora, lora_scale=2.0)
    eng.set_prefix([(k.cuda().half(), v.cuda().half()) for k, v in kv], valid)
    got = eng.predict(state, noise, state_mask=sm, action_mask=am).float().cpu()
    eng.check_status()
    assert float((got - want).abs().max()) < 5e-2 * max(1.0, float(want.abs().max()))
    # without the LoRA delta the answer differs
    plain = r.TorchRhinoVLA(cfg, sd, device="cuda").sample_actions(kv, valid, state, sm, noise, am, r.default_cond_table(cfg, 10)).cpu()
    assert float((plain - want).abs().max()) > 10 * float((got - want).abs().max())
