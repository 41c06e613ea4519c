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
