"""Pi0.5 engine (packed prefix, precomputed adaRMS schedule, graph-captured denoise loop) against the
padded/masked fp32 PyTorch formulation of the same model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(cfg, B, seed=0):
    g = torch.Generator().manual_seed(seed)
    s = cfg.vision.image_size
    images = torch.randn(B, cfg.num_views, 3, s, s, generator=g)
    image_mask = torch.ones(B, cfg.num_views, dtype=torch.bool)
    L = cfg.max_lang_tokens - 3
    tokens = torch.randint(0, cfg.vocab_size, (B, L), generator=g)
    n_lang = torch.tensor([L - 2 * b for b in range(B)])
    token_mask = torch.arange(L)[None] < n_lang[:, None]
    if B > 1:
        image_mask[1, 0] = False                    # a missing camera: its rows are absent from the packed prefix
    noise = torch.randn(B, cfg.horizon, cfg.action_dim, generator=g)
    return images, image_mask, tokens, token_mask, noise


@pytest.mark.parametrize("form", ["decode", "block"])
@pytest.mark.parametrize("B", [1, 5])
def test_suffix_attention_forms(B, form):
    """Both launch forms of the action rows' attention (one-token sequences on the decode kernel; one bidirectional
    query block per sample on the prefill kernel) against the fp32 formulation; ``auto`` picks by sample count."""
    from rhinoforge_b200.models.pi05 import Pi05Engine, TorchPi05, random_pi05_state_dict, tiny_pi05_config
    cfg = tiny_pi05_config()
    sd = random_pi05_state_dict(cfg, dtype=torch.float32, std=0.08, seed=3)
    args = _inputs(cfg, B, seed=2)
    want = TorchPi05(cfg, sd, device="cuda").sample_actions(*args, num_steps=4).cpu()
    eng = Pi05Engine(cfg, sd, max_batch=B)
    assert eng.suffix_attn == "auto"
    eng.suffix_attn = form
    for use_graph in (False, True):
        got = eng.predict(*args, num_steps=4, use_graph=use_graph).float().cpu()
        eng.check_status()
        assert float((got - want).abs().max() / want.abs().max()) < 3e-2, (form, use_graph)
    eng.close()


@pytest.mark.parametrize("B,steps", [(1, 10), (3, 4)])
def test_actions_match_fp32_reference(B, steps):
    from rhinoforge_b200.models.pi05 import Pi05Engine, TorchPi05, random_pi05_state_dict, tiny_pi05_config
    cfg = tiny_pi05_config()
    sd = random_pi05_state_dict(cfg, dtype=torch.float32, std=0.08, seed=3)
    args = _inputs(cfg, B)
    want = TorchPi05(cfg, sd, device="cuda").sample_actions(*args, num_steps=steps).cpu()
    eng = Pi05Engine(cfg, sd, max_batch=B)
    eager = eng.predict(*args, num_steps=steps, use_graph=False).float().cpu().clone()
    eng.check_status()
    rel = float((eager - want).abs().max() / want.abs().max())
    assert rel < 3e-2, rel
    built = eng.predict(*args, num_steps=steps).float().cpu().clone()        # BUILD
    replay = eng.predict(*args, num_steps=steps).float().cpu().clone()       # REPLAY
    eng.check_status()
    assert torch.equal(built, replay), "graph replay must be deterministic"
    assert float((replay - want).abs().max() / want.abs().max()) < 3e-2
    # a different prompt through the same graph: metadata buffers are updated in place
    args2 = _inputs(cfg, B, seed=5)
    want2 = TorchPi05(cfg, sd, device="cuda").sample_actions(*args2, num_steps=steps).cpu()
    import ctypes
    from rhinoforge_b200 import _native as N
    lib = N.lib()
    lib.rf_launch_count.restype = ctypes.c_uint64
    c0 = lib.rf_launch_count()
    got2 = eng.predict(*args2, num_steps=steps).float().cpu()
    assert lib.rf_launch_count() == c0, "vision tower, prefix prefill and denoise loop all replay from graphs"
    assert len(eng._prefill_graphs) == 1 and len(eng._graphs) == 1
    assert float((got2 - want2).abs().max() / want2.abs().max()) < 3e-2
    # another input geometry (camera 1 of sample 0 missing) builds its own prefill graph and stays correct
    im3 = args2[1].clone()
    im3[0, 1] = False
    args3 = (args2[0], im3, *args2[2:])
    want3 = TorchPi05(cfg, sd, device="cuda").sample_actions(*args3, num_steps=steps).cpu()
    got3 = eng.predict(*args3, num_steps=steps).float().cpu()
    assert len(eng._prefill_graphs) == 2
    assert float((got3 - want3).abs().max() / want3.abs().max()) < 3e-2
    eng.close()


def test_schedule_matches_per_step_dense():
    from rhinoforge_b200.models.pi05 import (EXP, Pi05Engine, conditioning_schedule, random_pi05_state_dict,
                                             tiny_pi05_config)
    import torch.nn.functional as F
    cfg = tiny_pi05_config()
    sd = random_pi05_state_dict(cfg, dtype=torch.float32, std=0.08, seed=4)
    eng = Pi05Engine(cfg, sd)
    sch = eng.schedule(5)
    cond = conditioning_schedule(sd, cfg, 5)
    b = f"{EXP}layers.2.post_attention_layernorm.dense."
    want = F.linear(cond[3], sd[b + "weight"], sd[b + "bias"])
    assert torch.allclose(sch["mod"][3, 2, 1, 0].float().cpu(), want, atol=2e-3, rtol=2e-2)
    assert sch["mod"].shape == (5, cfg.expert.layers, 2, 1, 3 * cfg.expert.hidden)
    eng.close()
