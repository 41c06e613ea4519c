"""Wall-OSS engine (Qwen2.5-VL prompt decoder + dense flow-matching action decoder over the shared KV cache) against
fp32 PyTorch: the prompt K/V and the greedy tokens come from the Hugging Face Qwen2.5-VL forward, the action decoder
from a plain statement of its math."""
import pytest
import torch

pytestmark = pytest.mark.gpu

IMG, VOCAB = 150, 200


def _tiny_vlm():
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VLForConditionalGeneration
    c = Qwen2_5_VLConfig(
        text_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=2,
                         num_key_value_heads=1, vocab_size=VOCAB, max_position_embeddings=512, rms_norm_eps=1e-6,
                         rope_parameters={"rope_type": "default", "rope_theta": 1e4, "mrope_section": [8, 12, 12]}),
        vision_config=dict(depth=3, hidden_size=160, num_heads=2, intermediate_size=216, patch_size=14, temporal_patch_size=2,
                           spatial_merge_size=2, out_hidden_size=128, window_size=56, fullatt_block_indexes=[1],
                           hidden_act="silu", tokens_per_second=1),
        image_token_id=IMG, video_token_id=151, vision_start_token_id=152, vision_end_token_id=153,
        tie_word_embeddings=False)
    c._attn_implementation = "eager"
    torch.manual_seed(0)
    m = Qwen2_5_VLForConditionalGeneration(c).float().eval()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * 0.06)
            elif "norm" in n and n.endswith("weight"):
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(0.05 * torch.randn(p.shape, generator=g))
    return c, m


def _to_wall_oss_names(hf_sd, layers: int, vis_depth: int):
    """Hugging Face Qwen2.5-VL tensors under the two-expert checkpoint's names (fused QKV / gate-up, per-expert norms)."""
    t, out = "model.language_model.", {}
    out["model.embed_tokens.weight"] = hf_sd[t + "embed_tokens.weight"]
    out["model.norms.0.weight"] = hf_sd[t + "norm.weight"]
    out["lm_head.weight"] = hf_sd["lm_head.weight"]
    for i in range(layers):
        s, d = f"{t}layers.{i}.", f"model.layers.{i}."
        for kind in ("weight", "bias"):
            out[d + f"self_attn.qkv_proj_experts.0.{kind}"] = torch.cat([hf_sd[s + f"self_attn.{x}_proj.{kind}"] for x in "qkv"], 0)
        out[d + "self_attn.o_proj_experts.0.weight"] = hf_sd[s + "self_attn.o_proj.weight"]
        out[d + "moe.experts.0.gate_up_proj.weight"] = torch.cat((hf_sd[s + "mlp.gate_proj.weight"], hf_sd[s + "mlp.up_proj.weight"]), 0)
        out[d + "moe.experts.0.down_proj.weight"] = hf_sd[s + "mlp.down_proj.weight"]
        out[d + "input_layernorms.0.weight"] = hf_sd[s + "input_layernorm.weight"]
        out[d + "post_attention_layernorms.0.weight"] = hf_sd[s + "post_attention_layernorm.weight"]
    for k, v in hf_sd.items():
        if k.startswith("model.visual.") and ".mlp.gate_proj." not in k and ".mlp.up_proj." not in k:
            out["visual." + k[len("model.visual."):]] = v
    for i in range(vis_depth):
        for kind in ("weight", "bias"):
            b = f"model.visual.blocks.{i}.mlp."
            out[f"visual.blocks.{i}.mlp.gate_up_proj.{kind}"] = torch.cat((hf_sd[b + f"gate_proj.{kind}"], hf_sd[b + f"up_proj.{kind}"]), 0)
    return out


def _prompt(grid):
    ids = [3, 9, 152] + [IMG] * int(grid[0].prod() // 4) + [153, 27, 152] + [IMG] * int(grid[1].prod() // 4) + [153, 81, 43, 129, 11]
    return torch.tensor(ids)


def _engine(hf_cfg, ref, cfg, exp_sd):
    from rhinoforge_b200.adapters.wall_oss import text_config
    from rhinoforge_b200.models.qwen25_vl_vision import Qwen25VLVisionConfig
    from rhinoforge_b200.models.wall_oss import WallOssEngine
    sd = _to_wall_oss_names(ref.state_dict(), cfg.layers, hf_cfg.vision_config.depth)
    sd.update(exp_sd)
    tc = hf_cfg.text_config
    flat = dict(vocab_size=VOCAB, hidden_size=tc.hidden_size, num_hidden_layers=tc.num_hidden_layers,
                num_attention_heads=tc.num_attention_heads, num_key_value_heads=tc.num_key_value_heads, rms_norm_eps=1e-6,
                rope_theta=1e4, rope_scaling={"mrope_section": [8, 12, 12]}, max_position_embeddings=512,
                experts=[dict(hidden_size=tc.hidden_size, intermediate_size=tc.intermediate_size),
                         dict(hidden_size=cfg.hidden, intermediate_size=cfg.inter)])
    return WallOssEngine(cfg, text_config(flat), Qwen25VLVisionConfig.from_hf(hf_cfg.vision_config), lambda n: sd[n],
                         names=set(sd), image_token_id=IMG, max_prefix=96, max_patches=128)


def _inputs():
    grid = torch.tensor([[1, 4, 6], [1, 4, 4]])
    g = torch.Generator().manual_seed(5)
    px = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 14 * 14, generator=g)
    return grid, px, _prompt(grid), g


def test_qwen25vl_prompt_decoder_matches_hf_tokens_and_logits():
    from rhinoforge_b200.models.wall_oss import random_wall_oss_expert, tiny_wall_oss_config
    hf_cfg, ref = _tiny_vlm()
    cfg = tiny_wall_oss_config()
    eng = _engine(hf_cfg, ref, cfg, random_wall_oss_expert(cfg, seed=3, dtype=torch.float32))
    grid, px, ids, _ = _inputs()
    tok, logits = eng.vlm.prefill(ids, px, grid, return_logits=True)
    with torch.no_grad():
        o = ref(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(ids[None] == IMG).int())
    want = o.logits[0, -1]
    got = logits.float().cpu().reshape(-1)[:VOCAB]
    assert float((got - want).abs().max()) < 3e-2 * max(1.0, float(want.abs().max()))
    assert int(tok.flatten()[0]) == int(want.argmax()) or float(want.topk(2).values.diff().abs()) < 2e-2
    eng.close()


@pytest.mark.parametrize("causal,masked,use_graph", [(True, False, True), (False, True, True), (True, True, False)])
def test_wall_oss_action_chunk_matches_fp32(causal, masked, use_graph):
    from rhinoforge_b200.models.wall_oss import TorchWallOssExpert, random_wall_oss_expert, tiny_wall_oss_config
    hf_cfg, ref = _tiny_vlm()
    cfg = tiny_wall_oss_config(causal_actions=causal)
    exp_sd = random_wall_oss_expert(cfg, seed=3, dtype=torch.float32)
    eng = _engine(hf_cfg, ref, cfg, exp_sd)
    grid, px, ids, g = _inputs()
    noise = torch.randn(cfg.horizon, cfg.action_dim, generator=g)
    dof = torch.ones(cfg.horizon, cfg.action_dim)
    pad = None
    if masked:
        dof[:, -2:] = 0.0
        dof[3:, 1] = 0.0                        # not row-constant
        pad = torch.randn(cfg.horizon, cfg.action_dim, generator=g) * 0.3
    got = eng.predict(ids, px, grid, noise, dof, padding_action=pad, use_graph=use_graph).float().cpu().clone()
    got2 = eng.predict(ids, px, grid, noise, dof, padding_action=pad, use_graph=use_graph).float().cpu().clone()
    eng.check_status()
    with torch.no_grad():
        o = ref(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(ids[None] == IMG).int(),
                use_cache=True)
    past = o.past_key_values
    layers = getattr(past, "layers", None)
    kv = [(layers[i].keys[0], layers[i].values[0]) if layers is not None else (past[i][0][0], past[i][1][0])
          for i in range(cfg.layers)]
    P, p0 = int(ids.numel()), int(eng.vlm._next_pos)
    oracle = TorchWallOssExpert(cfg, exp_sd)
    want = oracle.sample_actions(kv, P, p0, noise, dof, padding_action=pad)
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert err < 3e-2 * max(1.0, scale), (err, scale)
    assert torch.equal(got, got2), "a second call on the same inputs must reproduce the first bit for bit"
    if masked:                                  # inactive dimensions end on the padding action
        assert float((got[:, -2:] - pad[:, -2:]).abs().max()) < 2e-2
    import dataclasses
    other = TorchWallOssExpert(dataclasses.replace(cfg, causal_actions=not causal), exp_sd).sample_actions(
        kv, P, p0, noise, dof, padding_action=pad)
    assert float((other - want).abs().max()) > 1e-4, "the action mask must matter"
    eng.close()
