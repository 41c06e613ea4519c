"""GR00T action head, host side: profile shapes, tables, subset ordering, oracle structure."""
import math

import pytest
import torch

from rhinoforge_b200.models import gr00t as g


def test_full_profile_geometry():
    cfg = g.Gr00tConfig()
    shapes = {n: s for n, s, _ in g.gr00t_shapes(cfg)}
    p = g.AP + "model.transformer_blocks."
    assert shapes[p + "0.attn1.to_k.weight"] == (1536, 2048) and shapes[p + "1.attn1.to_k.weight"] == (1536, 1536)
    assert shapes[p + "31.norm1.linear.weight"] == (3072, 1536)
    assert shapes[g.AP + "action_encoder.W2.W"] == (32, 3072, 1536)
    assert shapes[g.AP + "vl_self_attention.transformer_blocks.3.ff.net.0.proj.weight"] == (8192, 2048)
    assert [cfg.bucket(s) for s in range(4)] == [0, 250, 500, 750]


def test_tables():
    cfg = g.tiny_gr00t_config()
    sd = g.random_gr00t_state_dict(cfg)
    c = g.timestep_cond(sd.__getitem__, cfg, 250)
    assert c.shape == (cfg.hidden,) and torch.isfinite(c).all()
    # bucket 0: cos-first sinusoid is [1..1 | 0..0]
    te = g.AP + "model.timestep_encoder.timestep_embedder."
    e0 = torch.cat((torch.ones(cfg.time_embed // 2), torch.zeros(cfg.time_embed // 2)))
    h = torch.nn.functional.silu(sd[te + "linear_1.weight"] @ e0 + sd[te + "linear_1.bias"])
    want = torch.nn.functional.silu(sd[te + "linear_2.weight"] @ h + sd[te + "linear_2.bias"])
    assert torch.allclose(g.timestep_cond(sd.__getitem__, cfg, 0), want, atol=1e-6)
    t = g.action_time_encoding(cfg, 500)
    half = cfg.hidden // 2
    assert abs(float(t[0]) - math.sin(500.0)) < 1e-4 and abs(float(t[half]) - math.cos(500.0)) < 1e-4


def test_subset_order():
    im = torch.tensor([0, 1, 1, 0, 1, 0, 0], dtype=torch.bool)
    ok = torch.tensor([1, 1, 1, 1, 0, 1, 0], dtype=torch.bool)
    order, nt, ni = g.subset_order(im, ok)
    assert order.tolist() == [0, 3, 5, 1, 2] and (nt, ni) == (3, 2)


def test_check_state_dict_reports():
    cfg = g.tiny_gr00t_config()
    sd = g.random_gr00t_state_dict(cfg)
    g.check_state_dict(cfg, sd.__getitem__)
    sd.pop(g.AP + "vlln.bias")
    sd[g.AP + "action_decoder.layer2.b"] = torch.zeros(cfg.embodiments, 5)
    with pytest.raises(ValueError, match="2 tensors") as e:
        g.check_state_dict(cfg, sd.__getitem__)
    assert "vlln.bias: missing" in str(e.value) and "action_decoder.layer2.b: (3, 5)" in str(e.value)


def test_oracle_cross_blocks_see_only_their_subset():
    cfg = g.tiny_gr00t_config()
    sd = g.random_gr00t_state_dict(cfg, seed=2)
    o = g.TorchGr00t(cfg, sd, embodiment=1)
    gen = torch.Generator().manual_seed(0)
    S = 9
    vl = torch.randn(S, cfg.vl_dim, generator=gen)
    im = torch.tensor([0, 0, 1, 1, 1, 0, 0, 1, 0], dtype=torch.bool)
    ok = torch.ones(S, dtype=torch.bool)
    ok[8] = False
    state, noise = torch.randn(cfg.state_dim, generator=gen), torch.randn(cfg.horizon, cfg.action_dim, generator=gen)
    a = o.denoise(vl, state, noise, im, ok)
    vl2 = vl.clone()
    vl2[8] += 3.0                                             # an invalid token never matters
    assert torch.allclose(a, o.denoise(vl2, state, noise, im, ok), atol=1e-6)
    vl3 = vl.clone()
    vl3[2] += 1.0
    assert not torch.allclose(a, o.denoise(vl3, state, noise, im, ok), atol=1e-4)
    assert a.shape == (cfg.horizon, cfg.action_dim)
    # another embodiment bank gives another answer
    assert not torch.allclose(a, g.TorchGr00t(cfg, sd, embodiment=0).denoise(vl, state, noise, im, ok), atol=1e-4)


def _bundle(tmp_path, cfg, extra=None, shards=2):
    from safetensors.torch import save_file
    import json
    sd = g.random_gr00t_state_dict(cfg, seed=7)
    sd.update(extra or {})
    names = sorted(sd)
    wmap = {}
    for i in range(shards):
        part = {n: sd[n].contiguous() for n in names[i::shards]}
        fn = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        save_file(part, str(tmp_path / fn))
        wmap.update({n: fn for n in part})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wmap}))
    return sd


def test_adapter_reader_and_config_inference(tmp_path):
    from rhinoforge_b200.adapters import gr00t as ad
    cfg = g.tiny_gr00t_config()
    sd = _bundle(tmp_path, cfg)
    get = ad.checkpoint_reader(str(tmp_path))
    assert get.names == set(sd) and torch.equal(get(g.AP + "vlln.weight"), sd[g.AP + "vlln.weight"])
    with pytest.raises(KeyError):
        get("nope")
    got = ad.head_config_from({"action_horizon": cfg.horizon, "num_inference_timesteps": cfg.steps,
                               "diffusion_model_cfg": {"num_attention_heads": cfg.heads, "attention_head_dim": cfg.head_dim},
                               "vl_self_attention_cfg": {"num_attention_heads": cfg.vl_heads}}, get)
    assert got == cfg
    from rhinoforge_b200.api.errors import UnsupportedModelError
    with pytest.raises(UnsupportedModelError, match="does not"):
        ad.head_config_from({"diffusion_model_cfg": {"num_attention_heads": 5, "attention_head_dim": 48}}, get)
    # without an index file the shards are scanned
    (tmp_path / "model.safetensors.index.json").unlink()
    assert ad.checkpoint_reader(str(tmp_path)).names == set(sd)


def test_backbone_getter_maps_prefix_and_ties_the_head():
    from rhinoforge_b200.adapters.gr00t import backbone_getter
    store = {"backbone.model.model.language_model.embed_tokens.weight": torch.ones(2, 2),
             "backbone.model.model.language_model.layers.0.self_attn.q_proj.weight": torch.zeros(1),
             "action_head.vlln.weight": torch.zeros(1)}
    get = store.__getitem__
    bg = backbone_getter(type("G", (), {"__call__": lambda s, n: get(n), "names": set(store)})())
    assert torch.equal(bg("lm_head.weight"), store["backbone.model.model.language_model.embed_tokens.weight"])
    assert "model.language_model.layers.0.self_attn.q_proj.weight" in bg.names and "lm_head.weight" in bg.names
    assert not any(n.startswith("action_head") for n in bg.names)
    with pytest.raises(ValueError, match="language-model tensors"):
        backbone_getter(type("G", (), {"__call__": lambda s, n: get(n), "names": {"action_head.vlln.weight"}})())


def test_get_action_validates_before_running():
    from rhinoforge_b200.adapters.gr00t import Gr00tN1d7VLA
    cfg = g.tiny_gr00t_config()
    ran = []

    class Text:
        max_tokens = 16
        hidden = torch.zeros(16, cfg.vl_dim)
        cache = type("C", (), {"max_seq_len": 32})()

        def check_status(self):
            ran.append("status")

    class Backbone:
        text = Text()

        def prefill(self, ids, px, grid):
            ran.append(("prefill", ids.numel()))

        def close(self):
            ran.append("bclose")

    class Head:
        max_vl = 16

        def __init__(self):
            self.cfg = cfg

        def vl_encode(self, h):
            return h

        def denoise(self, vl, state, noise, im, valid):
            ran.append(("denoise", vl.shape[0], int(im.sum()), state.numel(), tuple(noise.shape)))
            return noise

        def check_status(self):
            pass

        def close(self):
            ran.append("hclose")

    rt = Gr00tN1d7VLA(Backbone(), Head(), image_token_id=9, embodiment_id=1)
    ids = torch.tensor([[1, 9, 9, 2, 3]])
    with pytest.raises(ValueError, match="num_steps"):
        rt.get_action({"input_ids": ids, "state": torch.zeros(4)}, num_steps=cfg.steps + 1)
    with pytest.raises(ValueError, match="exceeds the built capacity"):
        rt.get_action({"input_ids": torch.zeros(1, 17, dtype=torch.long), "state": torch.zeros(4)})
    with pytest.raises(ValueError, match="padded"):
        rt.get_action({"input_ids": ids, "attention_mask": torch.tensor([[1, 1, 1, 1, 0]]), "state": torch.zeros(4)})
    with pytest.raises(ValueError, match="state has"):
        rt.get_action({"input_ids": ids, "state": torch.zeros(cfg.state_dim + 1)})
    assert [r for r in ran if r != ("prefill", 5)] == []
    ran.clear()
    a = rt.get_action({"input_ids": ids, "state": torch.zeros(4)}, seed=3)
    b = rt.get_action({"input_ids": ids, "state": torch.zeros(4)}, seed=3)
    assert a.shape == (1, cfg.horizon, cfg.action_dim) and torch.equal(a, b)
    assert ("denoise", 5, 2, cfg.state_dim, (cfg.horizon, cfg.action_dim)) in ran
    rt.close()
    assert ran[-2:] == ["hclose", "bclose"]
