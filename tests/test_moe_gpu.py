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


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_native_stack_layer_with_moe_mlp(dtype):
    """The stack executor's MoE branch (router GEMM, top-k, expert bank as one GLU GEMM, routing-weight block scale, one
    down GEMM with the residual) against the sparse fp32 evaluation.  The attention output projection is zero, so the
    layer reduces to ``x + moe(rmsnorm(x))``."""
    from rhinoforge_b200.models.moe import MoEConfig, MoEMLP, moe_reference
    from rhinoforge_b200.runtime.stack import NativeStack, StackSpec
    torch.manual_seed(2)
    H, E, I, S, T = 128, 16, 64, 64, 70
    cfg = MoEConfig(hidden=H, experts=E, top_k=4, expert_inter=I, shared_inter=S, routed_scale=2.5)
    sd = {"router.weight": torch.randn(E, H) * 0.3, "router.bias": torch.randn(E) * 0.05}
    for e in range(E):
        for n, shape in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
            sd[f"experts.{e}.{n}.weight"] = torch.randn(shape) * 0.08
    for n, shape in (("gate_proj", (S, H)), ("up_proj", (S, H)), ("down_proj", (H, S))):
        sd[f"shared.{n}.weight"] = torch.randn(shape) * 0.08
    sd = {k: v.cuda().to(dtype) for k, v in sd.items()}
    sd["router.bias"] = sd["router.bias"].float()
    bank = MoEMLP(cfg, sd, dtype=dtype)                     # builds the side-by-side expert bank
    norm_w = (1.0 + 0.1 * torch.randn(H, device="cuda")).to(dtype)
    inter = E * I + S
    lw = dict(norm1_w=torch.ones(H), wqkv=torch.randn(3 * 2 * 64, H) * 0.05, wo=torch.zeros(H, 2 * 64), norm2_w=norm_w,
              w_up=bank.w_gate_up, w_down=bank.w_down, moe_router_w=sd["router.weight"], moe_router_bias=sd["router.bias"])
    spec = StackSpec(layers=1, hidden=H, heads=2, kv_heads=2, head_dim=64, inter=inter, norm="rms", mlp="swiglu",
                     paged_kv=False, causal=False, max_tokens=128, max_seqs=4, moe_experts=E, moe_top_k=4,
                     moe_expert_inter=I, moe_routed_scale=2.5)
    stack = NativeStack(spec, [lw], dtype=dtype)
    x = (torch.randn(T, H, device="cuda") * 0.5).to(dtype)
    hidden = x.clone()
    lens = torch.tensor([40, 30], dtype=torch.int32, device="cuda")
    starts = torch.tensor([0, 40], dtype=torch.int32, device="cuda")
    stack.forward(hidden, q_start=starts, q_len=lens, kv_len=lens, max_q_len=40, max_kv_len=40,
                  pos=torch.zeros(T, dtype=torch.int32, device="cuda"))
    stack.check_status()
    xf = x.float()
    xn = (norm_w.float() * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6))).to(dtype)
    want = xf + moe_reference(cfg, sd, xn)
    rel = float((hidden.float() - want).abs().max() / want.abs().max())
    assert rel < (2e-2 if dtype == torch.float16 else 6e-2), rel
    stack.close()


def _moe_reference_by_expert(cfg, sd, x):
    """fp32 sparse MoE evaluated expert by expert (the same math as ``moe_reference``, without a Python loop per token)."""
    import torch.nn.functional as F
    g = lambda n: sd[n].float()
    xf = x.float()
    logits = (xf @ g("router.weight").t()).to(x.dtype).float()
    sc = torch.sigmoid(logits)
    top = torch.topk(sc + sd["router.bias"].float(), cfg.top_k, dim=-1).indices
    w = torch.gather(sc, 1, top)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * cfg.routed_scale
    mlp = lambda p, t: (F.silu(t @ g(p + "gate_proj.weight").t()) * (t @ g(p + "up_proj.weight").t())) @ g(p + "down_proj.weight").t()
    out = mlp("shared.", xf) if cfg.shared_inter else torch.zeros(x.shape[0], cfg.hidden, device=x.device)
    for e in range(cfg.experts):
        rows, pick = (top == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += w[rows, pick][:, None] * mlp(f"experts.{e}.", xf[rows])
    return out


@pytest.mark.parametrize("T", [50, 4096])
def test_moe_grouped_gemm_equals_sparse_reference(T):
    """Grouped form: picks bucketed by expert, rows gathered in expert order, one persistent launch per projection
    that reads only the picked experts' weights, combine in pick order.  T = 50 (a few rows per expert, every row
    block mostly padding) and T = 4096 (several row blocks per expert); the dense-einsum form must agree too."""
    from rhinoforge_b200.models.moe import MoEConfig, MoEMLP
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(3)
    E, H, I = 32, 256, 128
    cfg = MoEConfig(hidden=H, experts=E, top_k=4, expert_inter=I, shared_inter=128, routed_scale=2.5)
    sd = {"router.weight": torch.randn(E, H) * 0.2, "router.bias": torch.randn(E) * 0.05}
    for e in range(E):
        for n, shape in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
            sd[f"experts.{e}.{n}.weight"] = torch.randn(shape) * 0.06
    for n, shape in (("gate_proj", (128, H)), ("up_proj", (128, H)), ("down_proj", (H, 128))):
        sd[f"shared.{n}.weight"] = torch.randn(shape) * 0.06
    sd = {k: v.cuda().half() for k, v in sd.items()}
    sd["router.bias"] = sd["router.bias"].float()
    x = (torch.randn(T, H, device="cuda") * 0.5).half()
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    mlp = MoEMLP(cfg, sd, dense_max_tokens=0)
    got = mlp.forward_grouped(x, status=status)
    want = _moe_reference_by_expert(cfg, sd, x)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, status.tolist()
    rel = float((got.float() - want).abs().max() / want.abs().max())
    assert rel < 2e-2, rel
    # bucketing: every pick has a distinct sorted row inside its expert's range
    logits = K.gemm(x, mlp.router_w)
    ids, w = K.moe_select(logits, 4, bias=mlp.router_b, scale=2.5)
    slot_of, token_of_slot, slot_w, tiles = K.moe_group(ids, w, E)
    torch.cuda.synchronize()
    assert sorted(slot_of.tolist()) == list(range(T * 4))
    assert torch.equal(token_of_slot[slot_of.long()].cpu(), torch.arange(T * 4, dtype=torch.int32) // 4)
    counts = torch.bincount(ids.flatten().long().cpu(), minlength=E)
    assert int(tiles[0]) == int(((counts + 127) // 128).sum())
    if T <= 256:
        dense = MoEMLP(cfg, sd)(x)
        assert float((dense.float() - got.float()).abs().max() / want.abs().max()) < 2e-2
