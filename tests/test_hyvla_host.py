"""Hy-Embodied VLA on the host: merger pooling, prefix assembly, suffix-encoder fold, RoPE base."""
import torch
import torch.nn.functional as F

from rhinoforge_b200.models.hyvla import (LM_HEAD, MERGER_P, assemble_prefix, folded_suffix_encoder, merger_pool,
                                          random_hyvla_state_dict, rope_tables, step_times, time_embedding, tiny_hyvla_config,
                                          HyVlaConfig)


def test_rope_base_and_times():
    cfg = HyVlaConfig()
    assert abs(cfg.rope_base / 1.115884e7 - 1.0) < 1e-4        # 10000 * 1000^(128/126)
    assert step_times(10)[:3] == [1.0, 0.9, 0.8] and len(step_times(10)) == 10
    cos, sin = rope_tables(tiny_hyvla_config(), 8)
    assert cos.shape == (8, 32) and torch.allclose(cos[0], torch.ones(32)) and torch.allclose(sin[0], torch.zeros(32))
    e = time_embedding(torch.tensor([0.5]), 8)
    assert e.shape == (1, 8) and torch.allclose(e[0, :4] ** 2 + e[0, 4:] ** 2, torch.ones(4), atol=1e-6)


def test_merger_pool_equals_the_member_wise_definition():
    cfg = tiny_hyvla_config(grid=3)
    sd = random_hyvla_state_dict(cfg, seed=1)
    D = cfg.vlm_hidden
    x = torch.randn(2, 36, D)
    got = merger_pool(sd, cfg, x)
    assert got.shape == (2, 9, D)
    p = lambda n: sd[MERGER_P + n]
    img = x[1].view(6, 6, D)
    for gy, gx in ((0, 0), (2, 1)):
        members = torch.stack([img[2 * gy + dy, 2 * gx + dx] for dy in (0, 1) for dx in (0, 1)])
        mean = members.mean(0, keepdim=True).expand(4, -1)
        sc = F.linear(F.gelu(F.linear(torch.cat((members, mean), -1), p("pooler.predictor.0.weight"), p("pooler.predictor.0.bias"))),
                      p("pooler.predictor.2.weight"), p("pooler.predictor.2.bias"))
        out = (members * torch.softmax(sc, 0)).sum(0)
        want = F.linear(F.gelu(out), p("proj2.weight"), p("proj2.bias"))
        assert torch.allclose(got[1, gy * 3 + gx], want, atol=1e-5)


def test_prefix_layout_and_encoder_fold():
    cfg = tiny_hyvla_config()
    sd = random_hyvla_state_dict(cfg, seed=2)
    g, D = cfg.grid, cfg.vlm_hidden
    imgs = [torch.randn(g * g, D), torch.randn(g * g, D)]
    lang = torch.tensor([3, 4, 5])
    rows, vis = assemble_prefix(cfg, sd[LM_HEAD], imgs, lang)
    per = g * (g + 1) + 2
    assert rows.shape == (2 + 2 * per + 3, D) and int(vis.sum()) == 2 * g * g
    tok = sd[LM_HEAD]
    assert torch.equal(rows[0], tok[cfg.tok_bos]) and torch.equal(rows[2], tok[cfg.tok_vision_start])
    assert torch.equal(rows[3], imgs[0][0]) and torch.equal(rows[3 + g], tok[cfg.tok_vision_split]) and not bool(vis[3 + g])
    assert torch.equal(rows[2 + per - 1], tok[cfg.tok_vision_end]) and torch.equal(rows[-1], tok[5])
    E = cfg.expert_hidden
    w, sb = folded_suffix_encoder(sd, cfg, 4)
    x = torch.randn(cfg.n_action, cfg.action_dim)
    for k, t in enumerate(step_times(4)):
        a = F.linear(x, sd["model.action_in_proj.weight"], sd["model.action_in_proj.bias"])
        te = time_embedding(torch.tensor([t]), E).expand(cfg.n_action, -1)
        want = F.linear(torch.cat((a, te), -1), sd["model.action_time_mlp_in.weight"], sd["model.action_time_mlp_in.bias"])
        assert float((x @ w.t() + sb[k] - want).abs().max()) < 1e-5
