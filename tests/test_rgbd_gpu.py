"""InternVLA-N1 RGB-D encoder and System-2 backbone on the accelerator."""
import pytest
import torch

from rhinoforge_b200.models import rgbd as R

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rgbd_encoder_matches_oracle(dtype):
    c = R.tiny_rgbd_config()
    sd = R.random_rgbd_state_dict(c, seed=1)
    g = torch.Generator().manual_seed(2)
    img, dep = torch.rand(2, 2, 56, 56, 3, generator=g), torch.rand(2, 2, 56, 56, 1, generator=g)
    want = R.TorchRgbdEncoder(c, sd)(img, dep)
    enc = R.RgbdEncoder(c, sd, max_batch=2, dtype=dtype)
    got = enc(img, dep).cpu()
    enc.check_status()
    tol = 3e-2 if dtype == torch.float16 else 1.5e-1
    assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max()))
    one = enc(img[:1], dep[:1]).cpu()
    assert float((one - got[:1]).abs().max()) < 1e-2
    enc.close()


def test_rgbd_full_profile():
    c = R.RgbdConfig()
    sd = R.random_rgbd_state_dict(c, seed=3)
    g = torch.Generator().manual_seed(4)
    img, dep = torch.rand(1, 2, 224, 224, 3, generator=g), torch.rand(1, 2, 224, 224, 1, generator=g) * 5.0
    want = R.TorchRgbdEncoder(c, sd, device="cuda")(img, dep).cpu()
    enc = R.RgbdEncoder(c, sd)
    got = enc(img, dep).cpu()
    enc.check_status()
    assert got.shape == (1, 32, 384) and torch.isfinite(got).all()
    assert float((got - want).abs().max()) < 5e-2 * max(1.0, float(want.abs().max()))
    enc.close()


def test_system2_backbone_reads_the_latent_rows():
    from test_wall_oss_gpu import IMG, _inputs, _tiny_vlm
    from rhinoforge_b200.adapters.internvla_n1.backbone import build_qwen25vl_backbone
    hf_cfg, ref = _tiny_vlm()
    grid, px, ids, _ = _inputs()
    with torch.no_grad():
        o = ref(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(ids[None] == IMG).int(),
                output_hidden_states=True)
    want = o.hidden_states[-1][:, -4:, :]
    sd = ref.state_dict()
    get = lambda n: sd[n]
    get.names = set(sd)
    bb = build_qwen25vl_backbone("", get_weight=get, hf_config=hf_cfg.to_dict(), strict=False, max_seq_len=128, max_patches=128)
    got = bb(ids, px, grid).cpu()
    assert got.shape == want.shape
    assert float((got - want).abs().max()) < 4e-2 * float(want.abs().max())
    # the same rows from caller-assembled embeddings and positions
    embeds, pos3 = bb.engine.prepare(ids, px, grid)
    got2 = bb.forward_embeds(embeds[None], pos3[:, None, :]).cpu()
    assert float((got2 - got).abs().max()) < 1e-2
    bb.close()
