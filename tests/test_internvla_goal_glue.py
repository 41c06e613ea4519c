"""InternVLA-N1 goal glue: the module equals a hand-written statement of the same computation and loads strictly."""
import pytest
import torch
import torch.nn.functional as F

from rhinoforge_b200.adapters.internvla_n1 import GoalGlue, build_goal_glue
from rhinoforge_b200.adapters.internvla_n1.goal_glue import load_goal_glue_state


def by_hand(g: GoalGlue, vlm_tokens: torch.Tensor) -> torch.Tensor:
    m, c = g.vlm_embed_mlp, g.goal_compressor
    x = m[4](F.relu(m[2](F.relu(m[0](vlm_tokens)))))
    B, S, E = x.shape
    H, hd = c.num_heads, E // c.num_heads
    x = x + c.token_positional_encoding.position_embedding.weight[:S][None]
    q = c.target_embedding.weight[None].expand(B, -1, -1) + c.query_positional_encoding.position_embedding.weight[:1][None]
    w, b = c.cross_attention.in_proj_weight, c.cross_attention.in_proj_bias
    split = lambda t: t.reshape(B, -1, H, hd).transpose(1, 2)
    qh, kh, vh = split(F.linear(q, w[:E], b[:E])), split(F.linear(x, w[E:2 * E], b[E:2 * E])), split(F.linear(x, w[2 * E:], b[2 * E:]))
    att = torch.softmax(qh @ kh.transpose(-1, -2) / hd ** 0.5, dim=-1) @ vh
    return c.cross_attention.out_proj(att.transpose(1, 2).reshape(B, -1, E))


def test_goal_glue_matches_the_hand_written_computation_and_loads_strictly(tmp_path):
    from safetensors.torch import save_file
    torch.manual_seed(0)
    src = GoalGlue().eval()
    tokens = torch.randn(2, 4, 3584)
    with torch.no_grad():
        out = src(tokens)
        assert out.shape == (2, 1, 384) and out.dtype == torch.float32
        assert torch.allclose(out, by_hand(src, tokens), atol=1e-5, rtol=1e-4)

    flat = {"vlm_embed_mlp." + k: v.half() for k, v in src.vlm_embed_mlp.state_dict().items()}
    flat.update({"goal_compressor." + k: v.half() for k, v in src.goal_compressor.state_dict().items()})
    flat["goal_compressor.positional_encoding.pe"] = torch.zeros(1000, 384)      # the unused table of older files
    flat["nav_head.unrelated.weight"] = torch.zeros(3)
    path = tmp_path / "navdp_head.safetensors"
    save_file({k: v.contiguous() for k, v in flat.items()}, str(path))
    glue = build_goal_glue(path)
    assert not glue.training and next(glue.parameters()).dtype == torch.float32 and next(glue.parameters()).device.type == "cpu"
    half = GoalGlue().eval()
    half.load_state_dict({k: v.half().float() for k, v in src.state_dict().items()})
    with torch.no_grad():
        assert torch.allclose(glue(tokens), half(tokens), atol=1e-6)
    with pytest.raises(ValueError, match="only device='cpu'"):
        build_goal_glue(path, device="cuda")
    with pytest.raises(ValueError, match=r"must have shape \(1000, 384\)"):
        load_goal_glue_state(GoalGlue(), {**flat, "goal_compressor.positional_encoding.pe": torch.zeros(10, 384)})
    missing = {k: v for k, v in flat.items() if k != "goal_compressor.target_embedding.weight"}
    with pytest.raises(RuntimeError, match="target_embedding"):
        load_goal_glue_state(GoalGlue(), missing)
    with pytest.raises(RuntimeError, match="Unexpected"):
        load_goal_glue_state(GoalGlue(), {**flat, "vlm_embed_mlp.6.weight": torch.zeros(1)})
