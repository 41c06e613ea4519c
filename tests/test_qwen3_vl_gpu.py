"""Qwen3-VL (vision tower + M-RoPE text + DeepStack) against Hugging Face fp32 on a tiny random model."""
import pytest
import torch

pytestmark = pytest.mark.gpu

IMG, VOCAB = 150, 200


def _tiny():
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
        tie_word_embeddings=False)
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


def _prompt():
    grid = torch.tensor([[1, 4, 6], [1, 4, 4]])
    ids = torch.tensor([[1, 2, 152] + [IMG] * 6 + [153, 4, 5, 152] + [IMG] * 4 + [153, 6, 7, 8]])
    px = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 16 * 16, generator=torch.Generator().manual_seed(2))
    return ids, grid, px


def test_prefill_logits_and_greedy_decode_match_hf():
    from rhinoforge_b200.models.qwen3_vl import Qwen3VLEngine
    c, ref = _tiny()
    ids, grid, px = _prompt()
    types = (ids == IMG).int()
    steps = 6
    with torch.no_grad():
        o = ref(input_ids=ids, pixel_values=px, image_grid_thw=grid, mm_token_type_ids=types, use_cache=True)
        want_logits = o.logits[0, -1]
        toks = [int(want_logits.argmax())]
        past, cur = o.past_key_values, ids
        for _ in range(steps - 1):
            o = ref(input_ids=torch.tensor([[toks[-1]]]), past_key_values=past, use_cache=True)
            toks.append(int(o.logits[0, -1].argmax()))
    sd = ref.state_dict()
    eng = Qwen3VLEngine(c, lambda n: sd[n], names=set(sd), max_seq_len=128, max_patches=64, max_prefill_tokens=64)
    first, logits = eng.prefill(ids[0], px, grid, return_logits=True)
    got = logits[0].float().cpu()
    rel = float((got - want_logits).abs().max() / want_logits.abs().max())
    assert rel < 3e-2, rel
    rest = eng.decode(steps - 1)
    eng.text.check_status()
    mine = [int(first[0])] + rest[0].tolist()
    # greedy paths agree while the fp32 top-2 margin is larger than the fp16 error
    assert mine[0] == toks[0]
    agree = sum(a == b for a, b in zip(mine, toks))
    assert agree >= steps - 1, (mine, toks)
    eng.close()


def test_text_only_prompt_and_text_continuation():
    from rhinoforge_b200.models.qwen3_vl import Qwen3VLEngine
    c, ref = _tiny()
    ids = torch.tensor([[3, 9, 27, 81, 43, 129, 11]])
    with torch.no_grad():
        want = ref(input_ids=ids, mm_token_type_ids=torch.zeros_like(ids, dtype=torch.int32)).logits[0, -1]
    sd = ref.state_dict()
    eng = Qwen3VLEngine(c, lambda n: sd[n], names=set(sd), max_seq_len=128, max_patches=64, max_prefill_tokens=64)
    _, lg = eng.prefill(ids[0, :4], return_logits=True)
    _, lg = eng.extend(ids[0, 4:], return_logits=True)           # chunked continuation gives the same last row
    rel = float((lg[0].float().cpu() - want).abs().max() / want.abs().max())
    assert rel < 3e-2, rel
    eng.close()
