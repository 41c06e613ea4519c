"""QwenPI05 on the host: hoisted modulation schedule against the per-step definition, mask, adapter admission."""
import pytest
import torch

from rhinoforge_b200.adapters.qwenpi05 import build_engine, config_from, expert_state_dict
from rhinoforge_b200.api import UnsupportedModelError
from rhinoforge_b200.models.qwenpi05 import (TorchQwenPI05, euler_times, modulation_schedule, random_qwenpi05_state_dict,
                                             suffix_mask_matrix, time_conditioning, tiny_qwenpi05_config)


def test_schedule_rows_equal_the_adaptive_norm_definition():
    cfg = tiny_qwenpi05_config()
    sd = random_qwenpi05_state_dict(cfg, seed=1, dtype=torch.float32)
    o = TorchQwenPI05(cfg, sd)
    assert euler_times(4) == [1.0, 0.75, 0.5, 0.25]
    cond = time_conditioning(sd, cfg, 4)
    mod, fin = modulation_schedule(sd, cfg, cond)
    assert mod.shape == (4, cfg.layers, 2, 3 * cfg.width) and fin.shape == (4, 3 * cfg.width)
    W = cfg.width
    h = torch.randn(5, W)
    for (k, l, j, name) in ((0, 0, 0, "input_layernorm"), (3, 2, 1, "post_attention_layernorm")):
        y, gate = o._ada(f"expert.layers.{l}.{name}", h, cond[k])
        m = mod[k, l, j]
        assert torch.allclose(o._rms(h) * (1 + m[:W]) + m[W:2 * W], y, atol=1e-5)
        assert torch.allclose(torch.tanh(gate), m[2 * W:], atol=1e-6)


def test_mask_and_positions():
    valid = torch.tensor([1, 1, 1, 0, 0], dtype=torch.bool)
    m = suffix_mask_matrix(valid, torch.tensor([1, 0, 1], dtype=torch.bool), 10)
    assert m.int().tolist() == [[1, 1, 1, 0, 0, 1, 0, 1, 0, 0], [1, 1, 1, 0, 0, 1, 1, 1, 0, 0], [1, 1, 1, 0, 0, 1, 0, 1, 0, 0]]


def test_adapter_names_and_admission():
    cfg = tiny_qwenpi05_config()
    sd = random_qwenpi05_state_dict(cfg, seed=2, dtype=torch.float32)
    esd = {k[len("expert."):].replace(".cond.", ".dense."): v for k, v in sd.items() if k.startswith("expert.")}
    isd = {k[len("io."):]: v for k, v in sd.items() if k.startswith("io.")}
    flat = expert_state_dict(esd, isd)
    assert set(flat) == set(sd) and all(torch.equal(flat[k], sd[k]) for k in sd)
    c = config_from(dict(width=1024, num_hidden_layers=10, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                         intermediate_size=4096), dict(action_dim=14, state_dim=14, action_horizon=30), prefix_layer_offset=18)
    assert (c.width, c.layers, c.heads, c.kv_heads, c.inter, c.action_dim, c.horizon, c.prefix_layer_offset) == \
        (1024, 10, 16, 8, 4096, 14, 30, 18)
    with pytest.raises(UnsupportedModelError, match="head_dim"):
        config_from(dict(width=96, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=48,
                         intermediate_size=64))
    bad = dict(sd)
    del bad["expert.layers.1.self_attn.k_norm.weight"]
    with pytest.raises(UnsupportedModelError, match="lacks 1 expert tensors"):
        build_engine(cfg, bad)
    bad = dict(sd)
    bad["io.action_out_proj.weight"] = torch.zeros(3, 3)
    with pytest.raises(UnsupportedModelError, match="has shape"):
        build_engine(cfg, bad)
