"""HALO on the host: embeddings, schedule, checkpoint names."""
import math

import pytest
import torch

from rhinoforge_b200.models.halo import (SUFFIX, HaloConfig, TorchHalo, euler_schedule, halo_shapes, random_halo_state_dict,
                                         sinusoidal_pos_embedding, timestep_embedding, tiny_halo_config)


def test_schedule_and_embeddings():
    ts, dts = euler_schedule(10)
    assert ts.numel() == 9 and torch.allclose(dts, torch.full((9,), 1 / 9)) and float(ts[0]) == 1.0
    with pytest.raises(ValueError):
        euler_schedule(1)
    cfg = HaloConfig()
    e = timestep_embedding(torch.tensor([0.5]), cfg)
    half = cfg.time_freq_dim // 2
    f = torch.exp(-math.log(1e4) * torch.arange(half) / half)
    assert torch.allclose(e[0, :half], torch.cos(0.5 * f)) and torch.allclose(e[0, half:], torch.sin(0.5 * f))
    p = sinusoidal_pos_embedding(torch.tensor([3]), cfg)
    h2 = cfg.hidden // 2
    f2 = torch.exp(torch.arange(h2) * -(math.log(1e4) / (h2 - 1)))
    assert torch.allclose(p[0, :h2], torch.sin(3 * f2), atol=1e-6) and torch.allclose(p[0, h2:], torch.cos(3 * f2), atol=1e-6)


def test_names_and_chunk_layout():
    cfg = tiny_halo_config()
    act, gen = {n for n, _, _ in halo_shapes(cfg, "act")}, {n for n, _, _ in halo_shapes(cfg, "gen")}
    assert "language_model.model.layers.0.self_attn.q_proj_moe_act.bias" in act and "language_model.model.norm_moe_act.weight" in act
    assert "language_model.model.layers.2.mlp_moe_gen.down_proj.weight" in gen and "latent_pos_embed.pos_embed" in gen
    assert "input_linear_layer.weight" in act and "vae2llm.weight" in gen and not (act & {"vae2llm.weight"})
    assert cfg.chunk_rows("act") == cfg.action_rows + 2 and cfg.chunk_rows("gen") == cfg.latent_rows + 2
    sd = random_halo_state_dict(cfg, "act", seed=0)
    rows = TorchHalo(cfg, sd, "act").input_rows(torch.zeros(cfg.action_rows, cfg.action_dim), 0.3, torch.arange(cfg.action_rows),
                                                torch.tensor([4, 5]))
    emb = sd["language_model.model.embed_tokens.weight"]
    assert rows.shape == (cfg.action_rows + 2, cfg.hidden) and torch.equal(rows[0], emb[4]) and torch.equal(rows[-1], emb[5])


def test_cfg_combine_rule():
    import pytest
    import torch
    from rhinoforge_b200.models.halo import cfg_combine
    g = torch.Generator().manual_seed(0)
    v, vt, vi = (torch.randn(6, 4, generator=g) for _ in range(3))
    assert cfg_combine(v, None, None, 1.0, 1.0) is v
    t = vt + 3.0 * (v - vt)
    both = vi + 1.5 * (t - vi)
    scale = (v.norm() / (both.norm() + 1e-8)).clamp(0.0, 1.0)
    assert torch.allclose(cfg_combine(v, vt, vi, 3.0, 1.5), both * scale, atol=1e-6)
    rows = (v.norm(dim=-1, keepdim=True) / (t.norm(dim=-1, keepdim=True) + 1e-8)).clamp(0.3, 1.0)
    assert torch.allclose(cfg_combine(v, vt, None, 3.0, 1.0, 0.3, "channel"), t * rows, atol=1e-6)
    with pytest.raises(ValueError, match="cfg_text"):
        cfg_combine(v, None, vi, 2.0, 1.0)
    with pytest.raises(ValueError, match="cfg_img"):
        cfg_combine(v, vt, None, 1.0, 2.0)
    with pytest.raises(NotImplementedError):
        cfg_combine(v, vt, vi, 2.0, 2.0, 0.0, "text_channel")
