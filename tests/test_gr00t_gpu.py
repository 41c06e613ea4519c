"""GR00T VL encoder and DiT denoise loop on the accelerator against the fp32 oracle."""
import pytest
import torch

from rhinoforge_b200.models import gr00t as g

pytestmark = pytest.mark.gpu


def _case(cfg, S, seed=0):
    gen = torch.Generator().manual_seed(seed)
    hidden = torch.randn(S, cfg.vl_dim, generator=gen) * 2.0
    im = torch.zeros(S, dtype=torch.bool)
    im[2:2 + S // 2] = True
    ok = torch.ones(S, dtype=torch.bool)
    ok[-1] = False
    state = torch.randn(cfg.state_dim, generator=gen)
    noise = torch.randn(cfg.horizon, cfg.action_dim, generator=gen)
    return hidden, im, ok, state, noise


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_vl_encoder_matches_oracle(dtype):
    cfg = g.tiny_gr00t_config()
    sd = g.random_gr00t_state_dict(cfg, seed=1)
    hidden, *_ = _case(cfg, 21)
    want = g.TorchGr00t(cfg, sd).vl_encode(hidden)
    eng = g.Gr00tEngine(cfg, sd.__getitem__, max_vl=32, dtype=dtype)
    got = eng.vl_encode(hidden.cuda()).float().cpu()
    eng.check_status()
    tol = 3e-2 if dtype == torch.float16 else 1.5e-1
    assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max()))
    # the post-norm form of the same input gives the same result
    w_rms = 1.0 + 0.1 * torch.randn(cfg.vl_dim, generator=torch.Generator().manual_seed(3))
    normed = hidden * torch.rsqrt(hidden.pow(2).mean(-1, keepdim=True) + 1e-6) * w_rms
    got2 = eng.vl_encode(normed.cuda(), inv_norm_weight=1.0 / w_rms).float().cpu()
    assert float((got2 - want).abs().max()) < 2 * tol * max(1.0, float(want.abs().max()))


def test_denoise_matches_oracle_and_one_graph_serves_every_length():
    cfg = g.tiny_gr00t_config()
    sd = g.random_gr00t_state_dict(cfg, seed=2)
    oracle = g.TorchGr00t(cfg, sd, embodiment=2)
    eng = g.Gr00tEngine(cfg, sd.__getitem__, embodiment=2, max_vl=32)
    results = []
    for S, seed in ((21, 0), (13, 1), (21, 0)):
        hidden, im, ok, state, noise = _case(cfg, S, seed)
        vl = oracle.vl_encode(hidden)
        want = oracle.denoise(vl, state, noise, im, ok)
        got = eng.denoise(vl.cuda(), state, noise, im, ok).cpu()
        eng.check_status()
        assert float((got - want).abs().max()) < 4e-2 * max(1.0, float(want.abs().max())), S
        results.append(got)
    assert torch.equal(results[0], results[2])
    hidden, im, ok, state, noise = _case(cfg, 21, 0)
    eager = eng.denoise(oracle.vl_encode(hidden).cuda(), state, noise, im, ok, use_graph=False).cpu()
    assert torch.equal(eager, results[0])
    with pytest.raises(ValueError, match="at least one text token"):
        eng.denoise(oracle.vl_encode(hidden).cuda(), state, noise, torch.ones(21, dtype=torch.bool), ok)


def test_full_profile_denoise():
    cfg = g.Gr00tConfig(embodiments=2, max_pos=64)
    sd = g.random_gr00t_state_dict(cfg, seed=5)
    sd = {k: v.half() for k, v in sd.items()}
    oracle = g.TorchGr00t(cfg, sd, embodiment=1, device="cuda")
    eng = g.Gr00tEngine(cfg, sd.__getitem__, embodiment=1, max_vl=256)
    hidden, im, ok, state, noise = _case(cfg, 148, 4)
    vl_want = oracle.vl_encode(hidden)
    vl = eng.vl_encode(hidden.cuda())
    assert float((vl.float() - vl_want).abs().max()) < 5e-2 * float(vl_want.abs().max())
    want = oracle.denoise(vl_want, state, noise, im, ok).cpu()
    got = eng.denoise(vl, state, noise, im, ok).cpu()
    eng.check_status()
    assert torch.isfinite(got).all()
    assert float((got - want).abs().max()) < 5e-2 * max(1.0, float(want.abs().max()))


def test_bundle_end_to_end_against_hf_backbone_and_oracle(tmp_path):
    """A tiny bundle on disk (``backbone.model.*`` + ``action_head.*``) through ``build_gr00t_vla``: the backbone's
    residual stream after the selected layer matches Hugging Face's hidden state, the action matches the oracle fed
    with that hidden state."""
    import json
    from safetensors.torch import save_file
    from test_qwen3_vl_gpu import _tiny, _prompt, IMG
    from rhinoforge_b200.adapters.gr00t import build_gr00t_vla
    hf_cfg, ref = _tiny()
    select = 3
    cfg = g.tiny_gr00t_config(vl_dim=hf_cfg.text_config.hidden_size)
    head_sd = g.random_gr00t_state_dict(cfg, seed=9)
    bundle = {k: v.contiguous() for k, v in head_sd.items()}
    for k, v in ref.state_dict().items():
        if k == "lm_head.weight" or any(k.startswith(f"model.language_model.layers.{i}.") for i in range(select, 4)):
            continue                                            # the bundle carries neither an output head nor the cut layers
        bundle["backbone.model." + k] = v.contiguous()
    ck = tmp_path / "bundle"
    ck.mkdir()
    save_file(bundle, str(ck / "model-00001-of-00001.safetensors"))
    (ck / "config.json").write_text(json.dumps({"action_head_cfg": {
        "action_horizon": cfg.horizon, "num_inference_timesteps": cfg.steps,
        "diffusion_model_cfg": {"num_attention_heads": cfg.heads, "attention_head_dim": cfg.head_dim},
        "vl_self_attention_cfg": {"num_attention_heads": cfg.vl_heads, "attention_head_dim": cfg.vl_head_dim}}}))
    qdir = tmp_path / "qwen3vl"
    hf_cfg.save_pretrained(str(qdir))
    ids, grid, px = _prompt()
    # the residual stream after layer `select - 1` INCLUDING that layer's DeepStack addition (what the next layer would
    # read): the last DeepStack tap of this tiny model sits on the cut layer, so record the stream where it is added
    lm = ref.model.language_model
    seen, orig = [], lm._deepstack_process

    def record(*a, **k):
        out = orig(*a, **k)
        seen.append(out)
        return out
    lm._deepstack_process = record
    with torch.no_grad():
        ref(input_ids=ids, pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(ids == IMG).int())
    lm._deepstack_process = orig
    assert len(seen) == 3
    want_hidden = seen[select - 1][0]
    rt = build_gr00t_vla(str(ck), str(qdir), embodiment_id=1, max_vl=64, select_layer=select, max_patches=64)
    inputs = {"input_ids": ids, "pixel_values": px, "image_grid_thw": grid, "state": torch.linspace(-1, 1, cfg.state_dim - 2)}
    got_hidden = rt.backbone_hidden(inputs).float().cpu()
    assert float((got_hidden - want_hidden).abs().max()) < 3e-2 * float(want_hidden.abs().max())
    oracle = g.TorchGr00t(cfg, head_sd, embodiment=1)
    noise = torch.randn(1, cfg.horizon, cfg.action_dim, generator=torch.Generator().manual_seed(5))[0]
    state = torch.nn.functional.pad(inputs["state"], (0, 2))
    want = oracle.denoise(oracle.vl_encode(want_hidden), state, noise, (ids[0] == IMG), torch.ones(ids.numel(), dtype=torch.bool))
    got = rt.get_action(inputs, seed=5)
    assert got.shape == (1, cfg.horizon, cfg.action_dim)
    assert float((got[0] - want).abs().max()) < 6e-2 * max(1.0, float(want.abs().max()))
    assert torch.equal(got, rt.get_action(inputs, seed=5))
    rt.close()
