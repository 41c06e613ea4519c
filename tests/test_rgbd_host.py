"""InternVLA-N1 RGB-D encoder, host side: position-table resampling, preprocessing, adapter strictness."""
import pytest
import torch

from rhinoforge_b200.models import rgbd as R


def test_resample_pos_embed():
    g = torch.Generator().manual_seed(0)
    pe = torch.randn(1, 1 + 36, 8, generator=g)
    assert torch.equal(R.resample_pos_embed(pe, 6), pe[0])                    # same grid: untouched
    out = R.resample_pos_embed(pe, 4)
    assert out.shape == (17, 8) and torch.equal(out[0], pe[0, 0])
    full = R.resample_pos_embed(torch.randn(1, 1 + 37 * 37, 16, generator=g), 16)
    assert full.shape == (257, 16)
    # a constant table stays constant under the bicubic resize
    const = torch.ones(1, 1 + 49, 4) * 0.7
    assert torch.allclose(R.resample_pos_embed(const, 5), torch.full((26, 4), 0.7), atol=1e-5)


def test_preprocess_and_oracle_shapes():
    c = R.tiny_rgbd_config()
    img, dep = torch.rand(2, 2, 56, 56, 3), torch.rand(2, 2, 56, 56, 1)
    ti, td = R.preprocess(img, dep, 56)
    assert ti.shape == td.shape == (4, 3, 56, 56)
    assert torch.allclose(ti[1, 0, 3, 5], (img[0, 1, 3, 5, 0] - 0.485) / 0.229, atol=1e-6)
    assert torch.equal(td[:, 0], td[:, 2]) and torch.equal(td[2, 0], dep[1, 0, :, :, 0])
    sd = R.random_rgbd_state_dict(c)
    o = R.TorchRgbdEncoder(c, sd)
    y = o(img, dep)
    assert y.shape == (2, c.queries, c.embed)
    y2 = o(img, dep * 0.5)
    assert not torch.allclose(y, y2, atol=1e-4)                               # the depth tower matters
    assert torch.allclose(o(img[:1], dep[:1]), y[:1], atol=1e-5)              # batch elements are independent


def test_adapter_prefix_and_strictness(tmp_path):
    from safetensors.torch import save_file
    from rhinoforge_b200.adapters.internvla_n1.rgbd import build_rgbd_encoder, rgbd_state_dict
    c = R.tiny_rgbd_config()
    sd = R.random_rgbd_state_dict(c)
    bundle = {"rgbd_encoder." + k: v.contiguous() for k, v in sd.items()}
    bundle["rgbd_encoder.rgb_model.mask_token"] = torch.zeros(1, c.hidden)      # present in DINOv2 checkpoints, unused
    bundle["decoder.layers.0.norm1.weight"] = torch.ones(4)                    # other parts of the head file are ignored
    got = rgbd_state_dict(bundle, c)
    assert set(got) == set(sd)
    with pytest.raises(ValueError, match="unexpected"):
        rgbd_state_dict({**bundle, "rgbd_encoder.extra.weight": torch.zeros(1)}, c)
    broken = dict(bundle)
    broken.pop("rgbd_encoder.project_layer.bias")
    with pytest.raises(ValueError, match="missing"):
        rgbd_state_dict(broken, c)
    with pytest.raises(ValueError, match="no `rgbd_encoder"):
        rgbd_state_dict({"a": torch.zeros(1)}, c)
    path = tmp_path / "navdp_head.safetensors"
    save_file(bundle, str(path))
    enc = build_rgbd_encoder(path, device="cpu", config=c)
    img, dep = torch.rand(1, 2, 56, 56, 3), torch.rand(1, 2, 56, 56, 1)
    assert torch.allclose(enc(img, dep), R.TorchRgbdEncoder(c, sd)(img, dep), atol=1e-6)


def test_backbone_preflight():
    from rhinoforge_b200.adapters.internvla_n1.backbone import PROFILE, preflight
    from rhinoforge_b200.api.errors import UnsupportedModelError
    ok = dict(text_config=dict(PROFILE), vision_config={})
    preflight(ok)
    with pytest.raises(UnsupportedModelError, match="geometry"):
        preflight(dict(text_config={**PROFILE, "hidden_size": 2048}, vision_config={}))
    preflight(dict(text_config={**PROFILE, "hidden_size": 2048}, vision_config={}), strict=False)
    with pytest.raises(UnsupportedModelError, match="vision_config"):
        preflight(dict(text_config=dict(PROFILE)))


def test_qwen25_text_config_from_plain_config():
    from types import SimpleNamespace
    from rhinoforge_b200.models.qwen25_vl import qwen25_text_config
    from rhinoforge_b200.runtime.errors import UnsupportedModelError
    tc = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=2, num_key_value_heads=1,
              vocab_size=200, max_position_embeddings=512, rms_norm_eps=1e-6, model_type="qwen2_5_vl_text",
              rope_parameters={"rope_type": "default", "rope_theta": 1e4, "mrope_section": [8, 12, 12]})
    c = qwen25_text_config(SimpleNamespace(**tc))
    assert c.mrope_section == (8, 12, 12) and not c.mrope_interleaved and c.attention_bias and not c.qk_norm
    import pytest
    with pytest.raises(UnsupportedModelError, match="mrope_section"):
        qwen25_text_config(SimpleNamespace(**{**tc, "rope_parameters": {"rope_type": "default", "rope_theta": 1e4}}))
