"""Hy-Embodied VLA host preprocessing: image gate and letter-box, prompt clean-up, prefix / suffix masks."""
import numpy as np
import pytest
import torch

from rhinoforge_b200.adapters.hy_vla import (CAMERA_ORDER, PrefixLayout, apply_visual_segment_mask, build_observation,
                                              make_att_2d_masks, prefix_masks, prepare_images, prepare_language,
                                              prepare_state, resize_with_pad, sample_noise, suffix_masks)
from rhinoforge_b200.adapters.hy_vla.preprocess import ASSISTANT_TAG


class WordTokenizer:
    """Whitespace tokenizer with the Hugging Face call shape; the assistant tag is one token."""

    def __init__(self):
        self.vocab = {"<pad>": 0, ASSISTANT_TAG: 1}
        self.calls = []

    def __call__(self, texts, padding, padding_side, truncation, max_length, return_tensors, add_special_tokens):
        assert (padding, padding_side, truncation, return_tensors, add_special_tokens) == (
            "max_length", "right", True, "pt", False)
        self.calls.append(texts[0])
        words = texts[0].replace(ASSISTANT_TAG, f" {ASSISTANT_TAG} ").split()
        ids = [self.vocab.setdefault(w, len(self.vocab)) for w in words][:max_length]
        mask = [1] * len(ids) + [0] * (max_length - len(ids))
        return {"input_ids": torch.tensor([ids + [0] * (max_length - len(ids))]), "attention_mask": torch.tensor([mask])}


def test_letterbox_geometry_truncates_and_centres():
    img = torch.rand(1, 3, 480, 640)
    out = resize_with_pad(img, 224, 224, pad_value=-5.0)
    assert out.shape == (1, 3, 224, 224)
    assert (out[:, :, :28] == -5).all() and (out[:, :, 196:] == -5).all() and (out[:, :, 28:196] != -5).all()
    tall = resize_with_pad(torch.rand(1, 3, 301, 100), 224, 224, pad_value=9.0)      # 224 x int(74.4) = 74 wide
    assert (tall[..., :75] == 9).all() and (tall[..., 75:149] != 9).all() and (tall[..., 149:] == 9).all()  # 75 | 74 | 75
    odd = resize_with_pad(torch.rand(1, 3, 100, 299), 224, 224, pad_value=9.0)       # 74 rows, 150 to pad evenly;
    assert (odd[:, :, 75:149] != 9).all()
    assert torch.equal(resize_with_pad(torch.ones(1, 3, 224, 224) * 0.25, 224, 224), torch.ones(1, 3, 224, 224) * 0.25)
    with pytest.raises(ValueError):
        resize_with_pad(torch.rand(3, 8, 8), 4, 4)


def test_image_gate_accepts_unambiguous_forms_only():
    rgb = (torch.rand(1, 3, 224, 224) * 255).to(torch.uint8)
    want = rgb.float() / 255 * 2 - 1
    forms = [rgb, rgb[0], rgb[0].permute(1, 2, 0), rgb.permute(0, 2, 3, 1), rgb[0].permute(1, 2, 0).numpy(),
             rgb.float() / 255, rgb.to(torch.int32)]
    for got in prepare_images(forms):
        assert got.shape == (1, 3, 224, 224) and torch.allclose(got, want, atol=1e-6)

    class Pil:
        def convert(self, mode):
            assert mode == "RGB"
            return rgb[0].permute(1, 2, 0).numpy()
    assert torch.allclose(prepare_images([Pil()])[0], want, atol=1e-6)
    unit = torch.rand(1, 3, 224, 224)
    assert torch.equal(prepare_images([unit])[0], unit * 2.0 - 1.0)                  # fp32 in [0, 1] passes untouched
    for bad, exc, msg in ((rgb.float(), ValueError, "not \\[0, 1\\]"), (unit * 2 - 1, ValueError, "not \\[0, 1\\]"),
                          (torch.rand(2, 3, 8, 8), ValueError, "batch of 2"), (torch.rand(8, 8), ValueError, "3 or 4"),
                          (torch.rand(1, 4, 8, 8), ValueError, "3 RGB"), (rgb > 3, ValueError, "bool"),
                          ("frame.png", TypeError, "unsupported frame type")):
        with pytest.raises(exc, match=msg):
            prepare_images([bad])
    bars = prepare_images([torch.full((3, 100, 200), 0.5)])[0]
    assert (bars[:, :, 0] == -1).all() and torch.allclose(bars[:, :, 112], torch.zeros(1, 3, 224))   # bars at -1


def test_prompt_cleanup_is_idempotent_in_the_assistant_tag():
    tok = WordTokenizer()
    a_ids, a_mask = prepare_language("  pick_up the\nred_block ", tok)
    b_ids, b_mask = prepare_language("pick_up the\nred_block " + ASSISTANT_TAG, tok)
    assert tok.calls[0] == tok.calls[1] == "pick up the red block" + ASSISTANT_TAG
    assert torch.equal(a_ids, b_ids) and torch.equal(a_mask, b_mask)
    assert a_ids.shape == (1, 64) and a_ids.dtype == torch.int64 and a_mask.dtype == torch.bool and int(a_mask.sum()) == 6
    short, m = prepare_language("a b c d e f", tok, max_length=4)
    assert short.shape == (1, 4) and m.all()


def test_state_padding():
    assert torch.equal(prepare_state(None), torch.zeros(1, 32))
    s = prepare_state([1.0, 2.0, 3.0], 8)
    assert s.tolist() == [[1, 2, 3, 0, 0, 0, 0, 0]] and s.dtype == torch.float32
    assert prepare_state(np.arange(32, dtype=np.float64)).shape == (1, 32)
    with pytest.raises(ValueError, match="more than max_state_dim"):
        prepare_state(torch.zeros(33))


def _visible_by_definition(pad, image_of_row):
    """Element-wise statement of the prefix mask: patches see exactly their own image's patches; every other pair is
    causal; padding sees and is seen by nothing."""
    n = pad.numel()
    out = torch.zeros(n, n, dtype=torch.bool)
    for i in range(n):
        for j in range(n):
            if not (pad[i] and pad[j]):
                continue
            pi, pj = image_of_row[i], image_of_row[j]
            out[i, j] = (pi == pj) if (pi >= 0 and pj >= 0) else (j <= i)
    return out


def test_prefix_layout_and_visual_mask_match_the_elementwise_definition():
    lay = PrefixLayout(3, 7, 64)
    assert (lay.rows_per_image, lay.total) == (58, 240)
    assert lay.image_body(0) == (3, 59) and lay.image_body(2) == (119, 175)
    assert lay.patch_rows(0)[:2] == [(3, 10), (11, 18)] and lay.patch_rows(1)[0] == (61, 68)
    lang = torch.zeros(1, 64, dtype=torch.bool)
    lang[:, :9] = True
    pad, att, mod, idx, full = prefix_masks(3, 7, lang)
    assert pad.shape == att.shape == mod.shape == (1, 240) and att.all()
    assert int(pad.sum()) == 240 - 55 and int(mod.sum()) == 3 * 49 and len(idx) == 21 and full == [(3, 59), (61, 117), (119, 175)]
    assert not mod[0, 10] and not mod[0, 2] and not mod[0, 59] and mod[0, 3]          # split, start and end markers
    mask = make_att_2d_masks(pad, att)
    assert torch.equal(mask[0], torch.tril(torch.ones(240, 240, dtype=torch.bool)) & pad[0][None] & pad[0][:, None])
    apply_visual_segment_mask(mask, idx, full)
    assert torch.equal(mask[0], _visible_by_definition(pad[0], lay.image_id()))
    assert mask[0, 3, 58 - 1 - 1] and not mask[0, 61, 3] and not mask[0, 3, 61] and mask[0, 10, 3] and not mask[0, 3, 10]
    with pytest.raises(NotImplementedError):
        apply_visual_segment_mask(mask, idx, full, isolation=True)
    two = prefix_masks(2, 7, lang)[0]
    assert two.shape == (1, 2 + 2 * 58 + 64)                                          # a missing camera shortens the prefix


def test_suffix_blocks_and_noise():
    pad, att, mod = suffix_masks(50)
    assert pad.all() and mod.all() and att[0].nonzero().flatten().tolist() == [0, 1]
    m = make_att_2d_masks(pad, att)[0]
    assert m[0, 0] and not m[0, 1:].any()                                             # the state row sees only itself
    assert m[1:, :].all()                                                             # action rows see state and each other
    pad2, att2, _ = suffix_masks(4, n_state_tokens=2)
    assert att2[0].tolist() == [True, False, True, False, False, False]
    a, b = sample_noise(seed=7), sample_noise(seed=7)
    state = torch.random.get_rng_state()
    sample_noise(seed=8)
    assert torch.equal(a, b) and a.shape == (1, 50, 32) and torch.equal(torch.random.get_rng_state(), state)
    with pytest.raises(ValueError):
        make_att_2d_masks(pad[0], att)


def test_build_observation_end_to_end():
    frames = [torch.rand(3, 480, 640), (torch.rand(480, 640, 3) * 255).to(torch.uint8), torch.rand(1, 3, 224, 224)]
    obs = build_observation(frames, "open the_drawer", WordTokenizer(), state=[0.1] * 14, noise_seed=3)
    assert len(CAMERA_ORDER) == 3 and [tuple(i.shape) for i in obs["images"]] == [(1, 3, 224, 224)] * 3
    assert obs["n_valid"] == 2 + 3 * 58 + 4
    assert obs["lang_tokens"].shape == (64,) and obs["prefill_mask"].shape == (240, 240)
    assert obs["modality_mask"].shape == (240,) and obs["state"].shape == (1, 32) and obs["noise"].shape == (1, 50, 32)
    pos = obs["prefill_pos"]
    assert pos[:obs["n_valid"]].tolist() == list(range(obs["n_valid"])) and (pos[obs["n_valid"]:] == obs["n_valid"] - 1).all()
    dm = obs["denoise_mask"]
    assert dm.shape == (51, 240 + 51)
    assert dm[:, :obs["n_valid"]].all() and not dm[:, obs["n_valid"]:240].any()       # all real prefix rows, no padding
    assert dm[0, 240] and not dm[0, 241:].any() and dm[1:, 240:].all()
    assert obs["suffix_pos"].tolist() == list(range(obs["n_valid"], obs["n_valid"] + 51))
    given = torch.zeros(1, 50, 32, dtype=torch.float64)
    assert build_observation(frames[:1], "x", WordTokenizer(), noise=given)["noise"].dtype == torch.float32
    assert torch.equal(build_observation(frames, "x", WordTokenizer(), noise_seed=3)["noise"], obs["noise"])
