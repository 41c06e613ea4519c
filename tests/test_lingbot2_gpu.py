"""LingBot-VLA-v2 engine (Qwen3-VL prefix + sparse-MoE flow-matching action expert over the shared KV cache) against
fp32 PyTorch: the prefix K/V come from the Hugging Face Qwen3-VL forward, the expert from a plain statement of its math."""
import pytest
import torch

pytestmark = pytest.mark.gpu

IMG, VOCAB = 150, 200


def _tiny_vlm():
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLConfig
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLForConditionalGeneration
    c = Qwen3VLConfig(
        text_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=2,
                         num_key_value_heads=1, head_dim=64, vocab_size=VOCAB, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 1e4, "mrope_section": [12, 10, 10],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=3, hidden_size=128, num_heads=2, intermediate_size=256, out_hidden_size=128,
                           num_position_embeddings=64, deepstack_visual_indexes=[0, 1, 2]),
        image_token_id=IMG, video_token_id=151, vision_start_token_id=152, vision_end_token_id=153,
        tie_word_embeddings=True)
    c._attn_implementation = "eager"
    torch.manual_seed(0)
    m = Qwen3VLForConditionalGeneration(c).float().eval()
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


@pytest.mark.parametrize("blocked_tail,use_graph", [(0, True), (3, False)])
def test_lingbot2_action_chunk_matches_fp32(blocked_tail, use_graph):
    from rhinoforge_b200.models.lingbot2 import (EXP_P, VLM_P, Lingbot2Engine, TorchLingbot2Expert, random_lingbot2_expert,
                                                 tiny_lingbot2_config)
    hf_cfg, ref = _tiny_vlm()
    cfg = tiny_lingbot2_config(blocked_tail=blocked_tail)
    exp_sd = random_lingbot2_expert(cfg, seed=3, dtype=torch.float32)
    vlm_sd = ref.state_dict()
    sd = {VLM_P + k: v for k, v in vlm_sd.items()}
    sd.update(exp_sd)
    eng = Lingbot2Engine(cfg, hf_cfg, lambda n: sd[n], names=set(sd), max_prefix=64, max_patches=64)
    # two cameras (4x6 and 4x4 patches -> 6 and 4 merged tokens) and a 7-token instruction
    grid = torch.tensor([[1, 4, 6], [1, 4, 4]])
    g = torch.Generator().manual_seed(5)
    px = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 16 * 16, generator=g)
    lang = torch.tensor([3, 9, 27, 81, 43, 129, 11])
    ids = eng.build_input_ids([6, 4], lang, vision_boundaries=True)
    state = torch.randn(cfg.state_dim, generator=g)
    noise = torch.randn(cfg.horizon, cfg.action_dim, generator=g)
    got = eng.predict(ids, px, grid, state, noise, use_graph=use_graph).float().cpu().clone()
    got2 = eng.predict(ids, px, grid, state, noise, use_graph=use_graph).float().cpu().clone()
    eng.check_status()
    # oracle: Hugging Face fp32 prefix K/V, then the expert in plain PyTorch
    with torch.no_grad():
        o = ref(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(ids[None] == IMG).int(),
                use_cache=True)
    past = o.past_key_values
    layers = getattr(past, "layers", None)
    kv = [(layers[i].keys[0], layers[i].values[0]) if layers is not None else (past[i][0][0], past[i][1][0])
          for i in range(cfg.layers)]
    S, p0 = int(ids.numel()), int(eng.vlm._next_pos)
    want = TorchLingbot2Expert(cfg, exp_sd).sample_actions(kv, S, p0, state, noise)
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert err < 3e-2 * max(1.0, scale), (err, scale)
    assert torch.equal(got, got2), "a second call on the same inputs must reproduce the first bit for bit"
    # the mask matters: with the tail rows visible the result differs
    if blocked_tail:
        import dataclasses
        open_cfg = dataclasses.replace(cfg, blocked_tail=0)
        other = TorchLingbot2Expert(open_cfg, exp_sd).sample_actions(kv, S, p0, state, noise)
        assert float((other - want).abs().max()) > 1e-4
    eng.close()
