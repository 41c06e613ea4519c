"""RhinoVLA expert, host side: LoRA merge, oracle mask semantics, adapter flattening."""
import pytest
import torch

from rhinoforge_b200.models import rhinovla as r


def test_merge_lora():
    g = torch.Generator().manual_seed(0)
    base = {"expert.layers.0.self_attn.q_proj.weight": torch.randn(8, 6, generator=g), "other.weight": torch.ones(2, 2)}
    lora = {"expert.layers.0.self_attn.q_proj.lora_A.weight": torch.randn(3, 6, generator=g),
            "expert.layers.0.self_attn.q_proj.lora_B.weight": torch.randn(8, 3, generator=g)}
    out = r.merge_lora(base, lora, scale=0.5)
    want = base["expert.layers.0.self_attn.q_proj.weight"] + 0.5 * lora["expert.layers.0.self_attn.q_proj.lora_B.weight"] @ \
        lora["expert.layers.0.self_attn.q_proj.lora_A.weight"]
    assert torch.allclose(out["expert.layers.0.self_attn.q_proj.weight"], want, atol=1e-6)
    assert out["other.weight"] is base["other.weight"] and set(out) == set(base)
    with pytest.raises(KeyError, match="lora_B"):
        r.merge_lora(base, {"expert.layers.0.self_attn.q_proj.lora_A.weight": torch.zeros(3, 6)})
    with pytest.raises(KeyError, match="no base weight"):
        r.merge_lora(base, {"x.lora_A.weight": torch.zeros(3, 6), "x.lora_B.weight": torch.zeros(8, 3)})
    with pytest.raises(ValueError, match="do not produce"):
        r.merge_lora(base, {"other.lora_A.weight": torch.zeros(3, 6), "other.lora_B.weight": torch.zeros(2, 3)})


def test_oracle_masks_and_direction():
    cfg = r.tiny_rhinovla_config()
    sd = r.random_rhinovla_state_dict(cfg, dtype=torch.float32, seed=1)
    o = r.TorchRhinoVLA(cfg, sd)
    g = torch.Generator().manual_seed(2)
    P = 5
    kv = [(torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g), torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g))
          for _ in range(cfg.layers)]
    valid = torch.ones(P, dtype=torch.bool)
    state, noise = torch.randn(cfg.state_dim, generator=g), torch.randn(cfg.horizon, cfg.action_dim, generator=g)
    am = torch.ones(cfg.horizon, cfg.action_dim)
    am[:, -2:] = 0
    cond = r.default_cond_table(cfg, 4)
    x = o.sample_actions(kv, valid, state, torch.ones(cfg.state_dim), noise, am, cond)
    assert float(x[:, -2:].abs().max()) == 0.0 and float(x[:, :-2].abs().max()) > 0
    # the state mask enters as a token offset: flipping it changes the result
    sm = torch.ones(cfg.state_dim)
    sm[0] = 0
    assert not torch.allclose(x, o.sample_actions(kv, valid, state, sm, noise, am, cond), atol=1e-5)
    assert r.step_times(4) == [0.0, 0.25, 0.5, 0.75] and cond.shape == (4, cfg.width)
    names = {n for n, _, _ in r.rhinovla_shapes(cfg)}
    assert "io.action_time_mlp_in.weight" in names and "io.time_mlp_in.weight" not in names


def test_adapter_flattens_modules_and_checks():
    from rhinoforge_b200.adapters import rhinovla as ad
    from rhinoforge_b200.api.errors import UnsupportedModelError
    cfg = r.tiny_rhinovla_config()
    sd = r.random_rhinovla_state_dict(cfg, dtype=torch.float32)
    expert = {k[len("expert."):].replace(".cond.", ".dense."): v for k, v in sd.items() if k.startswith("expert.")}
    io = {k[len("io."):]: v for k, v in sd.items() if k.startswith("io.") and "_mask_proj" not in k}
    lin = lambda n: torch.nn.Linear(sd[f"io.{n}.weight"].shape[1], sd[f"io.{n}.weight"].shape[0])
    masks = {"state_mask_proj": lin("state_mask_proj"), "action_mask_proj": lin("action_mask_proj")}
    flat = ad.expert_state_dict(expert, io, masks)
    assert set(flat) == set(sd)
    got = ad.config_from(flat, heads=cfg.heads, kv_heads=cfg.kv_heads, horizon=cfg.horizon, rope_theta=cfg.rope_theta,
                         num_steps=cfg.num_steps)
    assert got == cfg
    ad.preflight(got, flat)
    broken = dict(flat)
    broken.pop("io.action_mask_proj.bias")
    with pytest.raises(UnsupportedModelError, match="1 tensors missing"):
        ad.preflight(got, broken)
    with pytest.raises(ValueError, match="suffix_len"):
        ad.build_rpu_expert(expert, action_io=io, mask_proj=masks, heads=cfg.heads, kv_heads=cfg.kv_heads, horizon=cfg.horizon,
                            suffix_len=99, device="cpu")
