"""MoE router and dense-einsum expert MLP against a token-by-token fp32 evaluation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("score_fn,E,k", [("sigmoid", 32, 4), ("softmax", 60, 8), ("sigmoid", 128, 6)])
def test_moe_select_matches_torch(score_fn, E, k):
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(0)
    T = 37
    logits = torch.randn(T, E, device="cuda").half()
    logits[3, 5] = logits[3, 9]                          # an exact tie goes to the lower index
    bias = torch.randn(E, device="cuda") * 0.1
    ids, w, dense = K.moe_select(logits, k, bias=bias, score_fn=score_fn, norm_topk=True, scale=2.5, dense=True)
    lf = logits.float()
    sc = torch.sigmoid(lf) if score_fn == "sigmoid" else torch.softmax(lf, -1)
    key = sc + bias
    order = torch.sort(key, dim=-1, descending=True, stable=True).indices[:, :k]
    assert torch.equal(ids.long(), order)
    ww = torch.gather(sc, 1, order)
    ww = ww / ww.sum(-1, keepdim=True) * 2.5
    assert torch.allclose(w, ww, atol=1e-4, rtol=1e-3)
    ref_dense = torch.zeros(T, E, device="cuda").scatter_(1, order, ww)
    assert torch.allclose(dense.float(), ref_dense, atol=2e-3, rtol=2e-3)


def test_moe_mlp_dense_einsum_equals_sparse_reference():
    from rhinoforge_b200.models.moe import MoEConfig, MoEMLP, moe_reference
    torch.manual_seed(1)
    cfg = MoEConfig(hidden=128, experts=32, top_k=4, expert_inter=64, shared_inter=128, routed_scale=4.0)
    sd = {"router.weight": torch.randn(32, 128) * 0.3, "router.bias": torch.randn(32) * 0.05}
    for e in range(32):
        for n, shape in (("gate_proj", (64, 128)), ("up_proj", (64, 128)), ("down_proj", (128, 64))):
            sd[f"experts.{e}.{n}.weight"] = torch.randn(shape) * 0.08
    for n, shape in (("gate_proj", (128, 128)), ("up_proj", (128, 128)), ("down_proj", (128, 128))):
        sd[f"shared.{n}.weight"] = torch.randn(shape) * 0.08
    sd = {k: v.cuda().half() for k, v in sd.items()}
    sd["router.bias"] = sd["router.bias"].float()
    x = (torch.randn(50, 128, device="cuda") * 0.5).half()
    got = MoEMLP(cfg, sd)(x)
    want = moe_reference(cfg, sd, x)
    rel = float((got.float() - want).abs().max() / want.abs().max())
    assert rel < 2e-2, rel
