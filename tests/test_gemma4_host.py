"""Gemma4 host side: rotary tables per layer type, admission."""
import pytest
import torch

from rhinoforge_b200.models.gemma4 import preflight, rope_tables
from rhinoforge_b200.runtime.errors import UnsupportedModelError

CFG = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=2, num_key_value_heads=1, head_dim=256,
           global_head_dim=512, sliding_window=16, layer_types=["sliding_attention", "sliding_attention", "full_attention"],
           num_kv_shared_layers=0, hidden_activation="gelu_pytorch_tanh",
           rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                            "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1000000.0}})


def test_rope_tables_match_hugging_face():
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig
    from transformers.models.gemma4.modeling_gemma4 import Gemma4TextRotaryEmbedding
    c = Gemma4TextConfig(**{**CFG, "vocab_size": 64, "max_position_embeddings": 64})
    rot = Gemma4TextRotaryEmbedding(c)
    pos = torch.arange(40)[None]
    for kind, hd in (("sliding_attention", 256), ("full_attention", 512)):
        cos, sin = rope_tables(c, kind, hd, 40)
        hc, hs = rot(torch.zeros(1, 1, 1), pos, layer_type=kind)
        assert cos.shape == (40, hd // 2)
        assert torch.allclose(cos, hc[0, :, :hd // 2], atol=1e-5) and torch.allclose(sin, hs[0, :, :hd // 2], atol=1e-5)
    # only a quarter of the global frequencies rotate
    cos, sin = rope_tables(CFG, "full_attention", 512, 8)
    assert float(sin[:, 64:].abs().max()) == 0.0 and float((cos[:, 64:] - 1).abs().max()) == 0.0 and float(sin[1:, :64].abs().min()) > 0


def test_preflight_rejects_what_is_not_built():
    geo = preflight(CFG)
    assert [g.head_dim for g in geo] == [256, 256, 512]
    for bad, word in ((dict(enable_moe_block=True), "mixture-of-experts"), (dict(hidden_activation="silu"), "activation"),
                      (dict(use_bidirectional_attention="all"), "bidirectional"), (dict(global_head_dim=384), "head_dim 384")):
        with pytest.raises(UnsupportedModelError, match=word):
            preflight({**CFG, **bad})
    with pytest.raises(UnsupportedModelError, match="rope_type"):
        rope_tables({**CFG, "rope_parameters": {"full_attention": {"rope_type": "yarn", "rope_theta": 1.0}}}, "full_attention", 512, 4)
