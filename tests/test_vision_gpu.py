"""Vision towers against the Hugging Face fp32 modules (random-init tiny configurations)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-6))


def _randomize(model, std=0.05, seed=0):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * std)
            elif "norm" in n and n.endswith("weight"):
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(0.1 * torch.randn(p.shape, generator=g))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_qwen3vl_vision_matches_hf(dtype):
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig as HFConfig
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionModel
    from rhinoforge_b200.models.vision import Qwen3VLVisionConfig, Qwen3VLVisionEncoder

    hc = HFConfig(depth=4, hidden_size=128, num_heads=2, intermediate_size=256, patch_size=16, temporal_patch_size=2,
                  spatial_merge_size=2, out_hidden_size=96, num_position_embeddings=64, deepstack_visual_indexes=[1, 2],
                  hidden_act="gelu_pytorch_tanh")
    hc._attn_implementation = "eager"
    ref = Qwen3VLVisionModel(hc).float().eval()
    _randomize(ref)
    grid = torch.tensor([[1, 4, 6], [1, 2, 2], [2, 4, 4]])
    T = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(T, 3 * 2 * 16 * 16, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        o = ref(px, grid_thw=grid)
    enc = Qwen3VLVisionEncoder(Qwen3VLVisionConfig.from_hf(hc), ref.state_dict(), dtype=dtype, max_patches=256)
    emb, deep = enc(px, grid)
    enc.tower.stack.check_status()
    tol = 2e-2 if dtype == torch.float16 else 6e-2
    assert emb.shape == o.pooler_output.shape
    assert _rel(emb, o.pooler_output) < tol
    assert len(deep) == 2
    for a, b in zip(deep, o.deepstack_features):
        assert _rel(a, b) < tol
    enc.close()


def test_siglip_matches_hf_with_padded_heads():
    from transformers import SiglipVisionConfig, SiglipVisionModel
    from rhinoforge_b200.models.vision import SiglipConfig, SiglipVisionEncoder

    hc = SiglipVisionConfig(hidden_size=144, intermediate_size=272, num_hidden_layers=3, num_attention_heads=2,
                            image_size=56, patch_size=14)          # head_dim 72 -> padded to 128, K = 588 -> 592
    hc._attn_implementation = "eager"
    ref = SiglipVisionModel(hc).float().eval()
    _randomize(ref)
    px = torch.randn(3, 3, 56, 56, generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = ref(pixel_values=px).last_hidden_state
    proj_w = torch.randn(64, 144, generator=torch.Generator().manual_seed(3)) * 0.05
    proj_b = torch.randn(64, generator=torch.Generator().manual_seed(4)) * 0.1
    enc = SiglipVisionEncoder(SiglipConfig.from_hf(hc), ref.state_dict(), max_images=4)
    got = enc(px)
    enc.tower.stack.check_status()
    assert got.shape == want.shape
    assert _rel(got, want) < 2e-2
    enc2 = SiglipVisionEncoder(SiglipConfig.from_hf(hc), ref.state_dict(), max_images=4, projector=(proj_w, proj_b))
    got2 = enc2(px)
    assert _rel(got2, want @ proj_w.T + proj_b) < 2e-2
    enc.close(); enc2.close()


def test_dinov3_matches_hf():
    from transformers import DINOv3ViTConfig, DINOv3ViTModel
    from rhinoforge_b200.models.vision import DINOv3Config, DINOv3Encoder

    hc = DINOv3ViTConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=2,
                         image_size=64, patch_size=16, num_register_tokens=4, layerscale_value=1.0)
    hc._attn_implementation = "eager"
    ref = DINOv3ViTModel(hc).float().eval()
    _randomize(ref)
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if "lambda1" in n:
                p.copy_(0.5 + 0.5 * torch.rand(p.shape, generator=torch.Generator().manual_seed(7)))
    px = torch.randn(2, 3, 64, 48, generator=torch.Generator().manual_seed(5))     # non-square: 4 x 3 patches
    with torch.no_grad():
        o = ref(pixel_values=px)
    enc = DINOv3Encoder(DINOv3Config.from_hf(hc), ref.state_dict(), max_images=2)
    last, pooled = enc(px)
    enc.tower.stack.check_status()
    assert last.shape == o.last_hidden_state.shape
    assert _rel(last, o.last_hidden_state) < 2e-2
    assert _rel(pooled, o.pooler_output) < 2e-2
    enc.close()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_qwen25vl_vision_matches_hf(dtype):
    """Window attention as varlen sequences in window-major order, full-attention blocks in between, head size 80 on
    padded heads, SwiGLU with biases and a padded intermediate size, merger, raster order restored."""
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig as HFConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel as HFModel
    from rhinoforge_b200.models.qwen25_vl_vision import Qwen25VLVisionConfig, Qwen25VLVisionEncoder

    hc = HFConfig(depth=5, hidden_size=160, num_heads=2, intermediate_size=216, patch_size=14, temporal_patch_size=2,
                  spatial_merge_size=2, out_hidden_size=96, window_size=56, fullatt_block_indexes=[1, 4], hidden_act="silu")
    hc._attn_implementation = "eager"
    ref = HFModel(hc).float().eval()
    _randomize(ref)
    grid = torch.tensor([[1, 6, 10], [2, 4, 4], [1, 8, 8]])
    T = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(T, 3 * 2 * 14 * 14, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(px, grid_thw=grid).pooler_output
    enc = Qwen25VLVisionEncoder(Qwen25VLVisionConfig.from_hf(hc), ref.state_dict(), dtype=dtype, max_patches=256)
    assert enc.segments == [(0, 1, False), (1, 2, True), (2, 4, False), (4, 5, True)]
    got = enc(px, grid)
    enc.tower.stack.check_status()
    assert got.shape == want.shape
    assert _rel(got, want) < (2e-2 if dtype == torch.float16 else 6e-2)
    enc.close()


def test_hyvit2_is_siglip_without_post_norm_from_timm_names():
    """HYViT2: timm-style checkpoint names, fused qkv, no post-LayerNorm, per-token projector on the last block's
    output.  Oracle: the Hugging Face SigLIP encoder's last hidden state *before* its post-LayerNorm."""
    from transformers import SiglipVisionConfig, SiglipVisionModel
    from rhinoforge_b200.models.vision import HYViT2Encoder, SiglipConfig

    hc = SiglipVisionConfig(hidden_size=144, intermediate_size=272, num_hidden_layers=3, num_attention_heads=2,
                            image_size=56, patch_size=14)
    hc._attn_implementation = "eager"
    ref = SiglipVisionModel(hc).float().eval()
    _randomize(ref)
    px = torch.randn(1, 3, 56, 56, generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = ref(pixel_values=px, output_hidden_states=True).hidden_states[-1]
    s = ref.state_dict()
    sd = {"patch_embed.proj.weight": s["vision_model.embeddings.patch_embedding.weight"],
          "patch_embed.proj.bias": s["vision_model.embeddings.patch_embedding.bias"],
          "pos_embed": s["vision_model.embeddings.position_embedding.weight"][None]}
    for i in range(3):
        a, b = f"vision_model.encoder.layers.{i}.", f"blocks.{i}."
        sd[b + "attn.qkv.weight"] = torch.cat([s[a + f"self_attn.{n}.weight"] for n in ("q_proj", "k_proj", "v_proj")])
        sd[b + "attn.qkv.bias"] = torch.cat([s[a + f"self_attn.{n}.bias"] for n in ("q_proj", "k_proj", "v_proj")])
        sd[b + "attn.proj.weight"], sd[b + "attn.proj.bias"] = s[a + "self_attn.out_proj.weight"], s[a + "self_attn.out_proj.bias"]
        for src, dst in (("layer_norm1", "norm1"), ("layer_norm2", "norm2"), ("mlp.fc1", "mlp.fc1"), ("mlp.fc2", "mlp.fc2")):
            sd[b + dst + ".weight"], sd[b + dst + ".bias"] = s[a + src + ".weight"], s[a + src + ".bias"]
    proj_w = torch.randn(64, 144, generator=torch.Generator().manual_seed(6)) * 0.05
    proj_b = torch.randn(64, generator=torch.Generator().manual_seed(7)) * 0.1
    enc = HYViT2Encoder(SiglipConfig.from_hf(hc), sd, projector=(proj_w, proj_b))
    got = enc(px)
    enc.tower.stack.check_status()
    assert _rel(got, want @ proj_w.T + proj_b) < 2e-2
    enc.close()
