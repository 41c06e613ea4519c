"""HALO mixture-of-transformers decoder (text weights on the two boundary rows, twin weights - with their own per-head
norms and biases - on the action / latent rows) as an action expert and as an image-flow step, against fp32 PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,use_graph", [("act", True), ("gen", True), ("act", False)])
def test_halo_rollout_matches_fp32(mode, use_graph):
    from rhinoforge_b200.models.halo import HaloEngine, TorchHalo, random_halo_state_dict, tiny_halo_config
    cfg = tiny_halo_config()
    sd = random_halo_state_dict(cfg, mode, seed=3)
    g = torch.Generator().manual_seed(5)
    P = 29
    kv = [(torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g) * 0.5, torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g) * 0.5)
          for _ in range(cfg.layers)]
    eng = HaloEngine(cfg, sd, mode, max_prefix=64)
    eng.set_prefix(kv, rope_position=11)
    body, width = eng.body, eng.width
    x0 = torch.randn(body, width, generator=g)
    pos_ids = torch.arange(body) if mode == "act" else torch.randint(0, cfg.max_latent_size ** 2, (body,), generator=g)
    text_ids = torch.tensor([7, 9])
    got = eng.rollout(x0, pos_ids, text_ids, num_timesteps=5, use_graph=use_graph).float().cpu().clone()
    got2 = eng.rollout(x0, pos_ids, text_ids, num_timesteps=5, use_graph=use_graph).float().cpu().clone()
    eng.check_status()
    oracle = TorchHalo(cfg, sd, mode)
    want = oracle.rollout(kv, 11, x0, pos_ids, text_ids, num_timesteps=5)
    assert float((got - want).abs().max()) < 3e-2 * max(1.0, float(want.abs().max()))
    assert torch.equal(got, got2)
    # the twin weights matter: an oracle that sends every row through the text set gives something else
    import copy
    sd_same = dict(sd)
    from rhinoforge_b200.models.halo import SUFFIX
    for k in list(sd):
        if SUFFIX[mode] in k:
            sd_same[k] = sd[k.replace(SUFFIX[mode], "")]
    other = TorchHalo(cfg, sd_same, mode).rollout(kv, 11, x0, pos_ids, text_ids, num_timesteps=5)
    assert float((other - want).abs().max()) > 1e-3
    eng.close()


@pytest.mark.parametrize("renorm", ["global", "channel"])
def test_halo_image_flow_with_guidance_branches(renorm):
    """Three prefix banks (cond / cfg_text / cfg_img) with their own lengths and rotary positions, text and image guidance,
    norm capping: against the fp32 statement of the same rule."""
    from rhinoforge_b200.models.halo import HaloEngine, TorchHalo, random_halo_state_dict, tiny_halo_config
    cfg = tiny_halo_config()
    sd = random_halo_state_dict(cfg, "gen", seed=4)
    g = torch.Generator().manual_seed(6)
    banks = []
    for P, rp in ((29, 31), (22, 24), (7, 8)):
        kv = [(torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g) * 0.5, torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g) * 0.5)
              for _ in range(cfg.layers)]
        banks.append((kv, rp))
    eng = HaloEngine(cfg, sd, "gen", max_prefix=64, branches=3)
    for b, (kv, rp) in enumerate(banks):
        eng.set_prefix(kv, rope_position=rp, branch=b)
    x0 = torch.randn(eng.body, eng.width, generator=g)
    pos_ids = torch.randint(0, cfg.max_latent_size ** 2, (eng.body,), generator=g)
    text_ids = torch.tensor([7, 9])
    kw = dict(cfg_text_scale=4.0, cfg_img_scale=1.5, cfg_renorm_min=0.1, cfg_renorm_type=renorm)
    got = eng.rollout(x0, pos_ids, text_ids, num_timesteps=4, **kw).float().cpu().clone()
    again = eng.rollout(x0, pos_ids, text_ids, num_timesteps=4, **kw).float().cpu().clone()
    eager = eng.rollout(x0, pos_ids, text_ids, num_timesteps=4, use_graph=False, **kw).float().cpu().clone()
    eng.check_status()
    oracle = TorchHalo(cfg, sd, "gen")
    want = oracle.rollout_cfg(banks, x0, pos_ids, text_ids, num_timesteps=4, **kw)
    assert float((got - want).abs().max()) < 4e-2 * max(1.0, float(want.abs().max()))
    assert torch.equal(got, again) and torch.equal(got, eager)
    plain = eng.rollout(x0, pos_ids, text_ids, num_timesteps=4).float().cpu().clone()
    assert float((plain - oracle.rollout(banks[0][0], banks[0][1], x0, pos_ids, text_ids, num_timesteps=4)).abs().max()) < 3e-2
    assert float((plain - got).abs().max()) > 1e-2                      # guidance changes the result
    # only text guidance: bank 2 is not needed
    eng2 = HaloEngine(cfg, sd, "gen", max_prefix=64, branches=2)
    eng2.set_prefix(*banks[0], branch=0)
    with pytest.raises(ValueError, match="prefix banks"):
        eng2.rollout(x0, pos_ids, text_ids, num_timesteps=4, cfg_text_scale=2.0)
    eng2.set_prefix(banks[1][0], banks[1][1], branch=1)
    t_only = eng2.rollout(x0, pos_ids, text_ids, num_timesteps=4, cfg_text_scale=2.0).float().cpu()
    want_t = oracle.rollout_cfg(banks, x0, pos_ids, text_ids, num_timesteps=4, cfg_text_scale=2.0)
    assert float((t_only - want_t).abs().max()) < 4e-2 * max(1.0, float(want_t.abs().max()))
    eng.close()
    eng2.close()
