"""Gated-DeltaNet kernels and the Qwen3.5 hybrid decoder against plain PyTorch / Hugging Face fp32."""
import os

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DT = [torch.float16, torch.bfloat16]


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-6))


@pytest.mark.parametrize("dt", DT)
def test_causal_conv1d_varlen_and_decode(dt):
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(0)
    Cc, lens = 264, [5, 70, 1, 2]
    T = sum(lens)
    x = torch.randn(T, Cc + 24, device="cuda").to(dt)          # wider pitch than C
    w = (torch.randn(Cc, 4, device="cuda") * 0.5).to(dt)
    state = torch.randn(6, 3, Cc, device="cuda").to(dt)
    slot = torch.tensor([4, 0, 2, 5], dtype=torch.int32, device="cuda")
    ql = torch.tensor(lens, dtype=torch.int32, device="cuda")
    qs = (torch.cumsum(ql, 0) - ql).to(torch.int32)
    st0 = state.clone()
    y = K.causal_conv1d(x[:, :Cc], w, state, q_start=qs, q_len=ql, max_q_len=max(lens), slot=slot)
    o = 0
    for i, L in enumerate(lens):
        full = torch.cat((st0[int(slot[i])].float(), x[o:o + L, :Cc].float()), 0)          # [3 + L, C]
        ref = F.silu(F.conv1d(full.t()[None], w.float()[:, None], groups=Cc)[0].t())
        assert _rel(y[o:o + L], ref) < (4e-3 if dt == torch.float16 else 2e-2)
        assert torch.equal(state[int(slot[i])].float(), full[-3:].to(dt).float())
        o += L
    # decode: one token per sequence, slot = sequence index
    xd = torch.randn(3, Cc, device="cuda").to(dt)
    st1 = state[:3].clone()
    yd = K.causal_conv1d(xd, w, state)
    full = torch.cat((st1.float(), xd.float()[:, None]), 1)                                  # [3, 4, C]
    ref = F.silu((full * w.float().t()[None]).sum(1))
    assert _rel(yd, ref) < (4e-3 if dt == torch.float16 else 2e-2)
    assert torch.equal(state[:3].float(), full[:, 1:].to(dt).float())


def _delta_rule_ref(q, k, v, b, a, A_log, dt_bias, S):
    """q,k [n,Hk,Dk], v [n,Hv,Dv], b,a [n,Hv], S [Hv,Dk,Dv] -> (o [n,Hv,Dv], S)."""
    n, Hk, Dk = q.shape
    Hv = v.shape[1]
    rep = Hv // Hk
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / Dk ** 0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(b)
    g = -torch.exp(A_log) * F.softplus(a + dt_bias)
    out = []
    for t in range(n):
        S = S * torch.exp(g[t])[:, None, None]
        kv = (S * k[t][:, :, None]).sum(1)
        d = (v[t] - kv) * beta[t][:, None]
        S = S + k[t][:, :, None] * d[:, None, :]
        out.append((S * q[t][:, :, None]).sum(1))
    return torch.stack(out), S


@pytest.mark.parametrize("dt", DT)
def test_gdn_recurrent_prefill_then_decode(dt):
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(1)
    Hk, Hv, Dk, Dv = 2, 4, 128, 64
    lens = [37, 3]
    T = sum(lens)
    width = 2 * Hk * Dk + Hv * Dv
    qkv = torch.randn(T, width, device="cuda").to(dt)
    ba = torch.randn(T, 16, device="cuda").to(dt)
    A_log = torch.log(torch.rand(Hv, device="cuda") * 4 + 0.5)
    dtb = torch.rand(Hv, device="cuda")
    state = torch.randn(3, Hv, Dk, Dv, device="cuda") * 0.1
    st0 = state.clone()
    slot = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
    fresh = torch.tensor([1, 0], dtype=torch.int32, device="cuda")
    ql = torch.tensor(lens, dtype=torch.int32, device="cuda")
    qs = (torch.cumsum(ql, 0) - ql).to(torch.int32)
    out = K.gdn_recurrent(qkv, ba[:, :8], ba[:, 8:], state, A_log, dtb, Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, q_start=qs, q_len=ql,
                          slot=slot, fresh=fresh)
    tol = 5e-3 if dt == torch.float16 else 3e-2
    o = 0
    for i, L in enumerate(lens):
        r = qkv[o:o + L].float()
        q, k = r[:, :Hk * Dk].view(L, Hk, Dk), r[:, Hk * Dk:2 * Hk * Dk].view(L, Hk, Dk)
        v = r[:, 2 * Hk * Dk:].view(L, Hv, Dv)
        S0 = torch.zeros_like(st0[0]) if int(fresh[i]) else st0[int(slot[i])]
        ref, S = _delta_rule_ref(q, k, v, ba[o:o + L, :Hv].float(), ba[o:o + L, 8:8 + Hv].float(), A_log, dtb, S0)
        assert _rel(out[o:o + L].view(L, Hv, Dv), ref) < tol
        assert _rel(state[int(slot[i])], S) < 1e-3
        o += L
    assert torch.equal(state[1], st0[1])          # untouched slot
    # decode step for two sequences, slots = sequence index
    qd = torch.randn(2, width, device="cuda").to(dt)
    bad = torch.randn(2, 16, device="cuda").to(dt)
    st1 = state.clone()
    od = K.gdn_recurrent(qd, bad[:, :8], bad[:, 8:], state, A_log, dtb, Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv)
    for s in range(2):
        r = qd[s:s + 1].float()
        ref, S = _delta_rule_ref(r[:, :Hk * Dk].view(1, Hk, Dk), r[:, Hk * Dk:2 * Hk * Dk].view(1, Hk, Dk),
                                 r[:, 2 * Hk * Dk:].view(1, Hv, Dv), bad[s:s + 1, :Hv].float(), bad[s:s + 1, 8:8 + Hv].float(),
                                 A_log, dtb, st1[s])
        assert _rel(od[s].view(Hv, Dv), ref[0]) < tol
        assert _rel(state[s], S) < 1e-3


@pytest.mark.parametrize("dt", DT)
def test_gdn_chunked_prefill_matches_recurrence(dt):
    """The block-parallel kernel against the fp32 token-by-token rule and the recurrent kernel: sequences that span several
    chunks and end inside one, a carried-in state, a one-token sequence, and a second call that continues from the state."""
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(3)
    Hk, Hv, Dk, Dv = 2, 4, 128, 64
    lens = [150, 64, 1, 71]
    T = sum(lens)
    width = 2 * Hk * Dk + Hv * Dv
    qkv = torch.randn(T, width, device="cuda").to(dt)
    ba = torch.randn(T, 16, device="cuda").to(dt)
    A_log = torch.log(torch.rand(Hv, device="cuda") * 4 + 0.5)
    dtb = torch.rand(Hv, device="cuda")
    state = torch.randn(5, Hv, Dk, Dv, device="cuda") * 0.1
    st0 = state.clone()
    slot = torch.tensor([3, 0, 4, 1], dtype=torch.int32, device="cuda")
    fresh = torch.tensor([1, 0, 0, 1], dtype=torch.int32, device="cuda")
    ql = torch.tensor(lens, dtype=torch.int32, device="cuda")
    qs = (torch.cumsum(ql, 0) - ql).to(torch.int32)
    kw = dict(Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, q_start=qs, q_len=ql, slot=slot, fresh=fresh)
    out = K.gdn_recurrent(qkv, ba[:, :8], ba[:, 8:], state, A_log, dtb, chunked=True, **kw)
    state_rec = st0.clone()
    out_rec = K.gdn_recurrent(qkv, ba[:, :8], ba[:, 8:], state_rec, A_log, dtb, **kw)
    tol = 5e-3 if dt == torch.float16 else 3e-2
    o = 0
    finals = {}
    for i, L in enumerate(lens):
        r = qkv[o:o + L].float()
        q, k = r[:, :Hk * Dk].view(L, Hk, Dk), r[:, Hk * Dk:2 * Hk * Dk].view(L, Hk, Dk)
        v = r[:, 2 * Hk * Dk:].view(L, Hv, Dv)
        S0 = torch.zeros_like(st0[0]) if int(fresh[i]) else st0[int(slot[i])]
        ref, S = _delta_rule_ref(q, k, v, ba[o:o + L, :Hv].float(), ba[o:o + L, 8:8 + Hv].float(), A_log, dtb, S0)
        assert _rel(out[o:o + L].view(L, Hv, Dv), ref) < tol, i
        assert _rel(state[int(slot[i])], S) < 1e-3, (i, _rel(state[int(slot[i])], S))
        finals[int(slot[i])] = S
        o += L
    assert _rel(out, out_rec) < tol and _rel(state, state_rec) < 1e-3
    assert torch.equal(state[2], st0[2])          # untouched slot
    # continue the first sequence from its stored state
    L2 = 80
    q2 = torch.randn(L2, width, device="cuda").to(dt)
    ba2 = torch.randn(L2, 16, device="cuda").to(dt)
    one = dict(Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, q_start=torch.zeros(1, dtype=torch.int32, device="cuda"),
               q_len=torch.tensor([L2], dtype=torch.int32, device="cuda"), slot=torch.tensor([3], dtype=torch.int32, device="cuda"),
               fresh=torch.zeros(1, dtype=torch.int32, device="cuda"))
    o2 = K.gdn_recurrent(q2, ba2[:, :8], ba2[:, 8:], state, A_log, dtb, chunked=True, **one)
    r = q2.float()
    ref, S = _delta_rule_ref(r[:, :Hk * Dk].view(L2, Hk, Dk), r[:, Hk * Dk:2 * Hk * Dk].view(L2, Hk, Dk), r[:, 2 * Hk * Dk:].view(L2, Hv, Dv),
                             ba2[:, :Hv].float(), ba2[:, 8:8 + Hv].float(), A_log, dtb, finals[3])
    assert _rel(o2.view(L2, Hv, Dv), ref) < tol and _rel(state[3], S) < 1e-3


def test_gdn_chunked_is_faster_than_token_serial_on_a_long_prompt():
    """Qwen3.5 geometry (16 key heads, 32 value heads of 128) over 4096 tokens: the chunked kernel has to beat the
    token-by-token kernel by a wide margin and leave the same state."""
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(4)
    Hk, Hv, Dk, Dv, T = 16, 32, 128, 128, 4096
    width = 2 * Hk * Dk + Hv * Dv
    qkv = torch.randn(T, width, device="cuda", dtype=torch.bfloat16)
    ba = torch.randn(T, 64, device="cuda", dtype=torch.bfloat16)
    A_log = torch.log(torch.rand(Hv, device="cuda") * 4 + 0.5)
    dtb = torch.rand(Hv, device="cuda")
    kw = dict(Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, q_start=torch.zeros(1, dtype=torch.int32, device="cuda"),
              q_len=torch.tensor([T], dtype=torch.int32, device="cuda"), slot=torch.zeros(1, dtype=torch.int32, device="cuda"),
              fresh=torch.ones(1, dtype=torch.int32, device="cuda"))
    times, states, outs = {}, {}, {}
    for chunked in (False, True):
        state = torch.zeros(1, Hv, Dk, Dv, device="cuda")
        for _ in range(2):
            outs[chunked] = K.gdn_recurrent(qkv, ba[:, :32], ba[:, 32:], state, A_log, dtb, chunked=chunked, **kw)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            K.gdn_recurrent(qkv, ba[:, :32], ba[:, 32:], state, A_log, dtb, chunked=chunked, **kw)
        e1.record()
        torch.cuda.synchronize()
        times[chunked] = e0.elapsed_time(e1) / 3
        states[chunked] = state.clone()
    print(f"gdn 4096 tokens: token-serial {times[False]:.3f} ms, chunked {times[True]:.3f} ms, x{times[False] / times[True]:.1f}")
    assert _rel(states[True], states[False]) < 1e-3, _rel(states[True], states[False])
    assert _rel(outs[True], outs[False]) < 3e-2
    assert times[True] * 5 < times[False], times


def test_small_gdn_helpers():
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(2)
    x = torch.randn(7, 4, 128, device="cuda", dtype=torch.float16)
    zfull = torch.randn(7, 4 * 128 + 64, device="cuda", dtype=torch.float16)
    w = (1 + 0.1 * torch.randn(128, device="cuda")).half()
    y = K.rmsnorm_gated(x.view(7, -1), zfull[:, 64:], w, 4, 1e-6)
    xf = x.float()
    n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).half().float()
    ref = w.float() * n * F.silu(zfull[:, 64:].float().view(7, 4, 128))
    assert _rel(y.view(7, 4, 128), ref) < 4e-3
    a = torch.randn(9, 256, device="cuda", dtype=torch.float16)
    g = torch.randn(9, 304, device="cuda", dtype=torch.float16)
    want = a.float() * torch.sigmoid(g[:, 40:296].float())
    K.sigmoid_gate(a, g[:, 40:296])
    assert _rel(a, want) < 2e-3
    c = torch.randn(5, 3, 64, device="cuda")
    assert torch.allclose(K.cumsum(c), c.cumsum(-1), atol=1e-5)
    c2 = torch.randn(6, 100, device="cuda")
    assert torch.allclose(K.cumsum(c2), c2.cumsum(-1), atol=1e-4)
    m = torch.randn(4, 64, 64, device="cuda") * 0.2
    inv = K.unit_tril_inv(m)
    eye = torch.eye(64, device="cuda")
    assert torch.allclose((eye - m.tril(-1)) @ inv, eye.expand(4, 64, 64), atol=1e-4)


def _tiny_hf():
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM
    c = Qwen3_5TextConfig(
        vocab_size=304, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=2,
        num_key_value_heads=1, head_dim=64, linear_conv_kernel_dim=4, linear_key_head_dim=128,
        linear_value_head_dim=128, linear_num_key_heads=2, linear_num_value_heads=4,
        layer_types=["linear_attention", "linear_attention", "full_attention", "linear_attention"],
        rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25,
                         "mrope_section": [3, 3, 2], "mrope_interleaved": True},
        max_position_embeddings=512, tie_word_embeddings=False)
    c._attn_implementation = "eager"
    m = Qwen3_5ForCausalLM(c).float().eval()
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * 0.06)
            elif n.endswith("A_log"):
                p.copy_(torch.log(torch.rand(p.shape, generator=g) * 4 + 0.5))
            elif n.endswith("dt_bias"):
                p.copy_(torch.rand(p.shape, generator=g))
            elif n.endswith("linear_attn.norm.weight"):
                p.copy_(1 + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(0.1 * torch.randn(p.shape, generator=g))
    return c, m


def test_qwen3_5_engine_matches_hf():
    from rhinoforge_b200.models.decoder import DecoderConfig
    from rhinoforge_b200.runtime.engine import DecoderEngine
    c, ref = _tiny_hf()
    ref = ref.cuda()              # on a GPU box the Hugging Face module picks device kernels: keep it on the device
    sd = ref.state_dict()
    cfg = DecoderConfig.from_hf(c)
    eng = DecoderEngine(cfg, lambda n: sd[n], max_batch=2, max_seq_len=128, max_prefill_tokens=32)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 304, (L,), generator=g) for L in (45, 9)]       # 45 > 32: chunked prefill carries state
    steps = 5
    want_tok, want_first = [], []
    with torch.no_grad():
        for p in prompts:
            o = ref(input_ids=p[None].cuda(), use_cache=True)
            want_first.append(o.logits[0, -1])
            toks = [int(o.logits[0, -1].argmax())]
            past = o.past_key_values
            for _ in range(steps - 1):
                o = ref(input_ids=torch.tensor([[toks[-1]]], device="cuda"), past_key_values=past, use_cache=True)
                toks.append(int(o.logits[0, -1].argmax()))
            want_tok.append(toks)
    first, logits = eng.prefill(prompts, return_logits=True)
    for b in range(2):
        assert _rel(logits[b], want_first[b]) < 3e-2
    rest = eng.decode(steps - 1)
    eng.check_status()
    for b in range(2):
        mine = [int(first[b])] + rest[b].tolist()
        assert mine[0] == want_tok[b][0]
        assert sum(x == y for x, y in zip(mine, want_tok[b])) >= steps - 1, (mine, want_tok[b])
    eng.close()


def test_qwen3_5_vision_path_matches_hf():
    """Image + text through the adapter's multimodal handle against Hugging Face ``Qwen3_5ForConditionalGeneration`` fp32:
    the ViT without DeepStack, image rows spliced into the embeddings, three-axis positions, the hybrid decoder."""
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5Config
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForConditionalGeneration
    from rhinoforge_b200.adapters.qwen3_5 import Qwen3_5Adapter
    from rhinoforge_b200.api.cache import RPUCache
    from rhinoforge_b200.runtime import live_handle
    IMG = 150
    c = Qwen3_5Config(
        text_config=dict(vocab_size=304, hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=2,
                         num_key_value_heads=1, head_dim=64, linear_conv_kernel_dim=4, linear_key_head_dim=128,
                         linear_value_head_dim=128, linear_num_key_heads=2, linear_num_value_heads=4,
                         layer_types=["linear_attention", "linear_attention", "full_attention", "linear_attention"],
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25,
                                          "mrope_section": [3, 3, 2], "mrope_interleaved": True},
                         max_position_embeddings=512),
        vision_config=dict(depth=3, hidden_size=128, num_heads=2, intermediate_size=256, out_hidden_size=128,
                           num_position_embeddings=64),
        image_token_id=IMG, video_token_id=151, vision_start_token_id=152, vision_end_token_id=153, tie_word_embeddings=False)
    c._attn_implementation = "eager"
    torch.manual_seed(0)
    ref = Qwen3_5ForConditionalGeneration(c).float().eval()
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * 0.06)
            elif n.endswith("A_log"):
                p.copy_(torch.log(torch.rand(p.shape, generator=g) * 4 + 0.5))
            elif n.endswith("dt_bias"):
                p.copy_(torch.rand(p.shape, generator=g))
            elif "norm" in n and n.endswith("weight"):
                p.copy_((1.0 if "visual" in n or "linear_attn.norm" in n else 0.0) + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(0.05 * torch.randn(p.shape, generator=g))
    grid = torch.tensor([[1, 4, 6], [1, 4, 4]])
    ids = torch.tensor([[1, 2, 152] + [IMG] * 6 + [153, 4, 5, 152] + [IMG] * 4 + [153, 6, 7, 8]])
    px = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 16 * 16, generator=torch.Generator().manual_seed(2))
    ref = ref.cuda()
    with torch.no_grad():
        want = ref(input_ids=ids.cuda(), pixel_values=px.cuda(), image_grid_thw=grid.cuda(),
                   mm_token_type_ids=(ids == IMG).int().cuda()).logits[0, -1].float().cpu()
    os.environ["RPU_QWEN3_5_ALLOW_ANY_PROFILE"] = "1"
    live_handle._reset_for_tests()
    c.rpu_use_vision = True
    sd = {k: v.cpu() for k, v in ref.state_dict().items()}
    get = lambda n: sd[n]
    get.names = set(sd)
    try:
        handle = Qwen3_5Adapter(None, config=c, get_weight=get, dtype=torch.float16).to_rpu(max_seq_len=128, max_patches=64)
        eng = handle.vl
        _, logits = eng.prefill(ids[0], px, grid, return_logits=True)
        got = logits[0].float().cpu()
        rel = float((got - want).abs().max() / want.abs().max())
        assert rel < 3e-2, rel
        # text continuation keeps the positions running after the images
        nxt = int(want.argmax())
        with torch.no_grad():
            ids2 = torch.cat((ids, torch.tensor([[nxt, 9]])), 1)
            want2 = ref(input_ids=ids2.cuda(), pixel_values=px.cuda(), image_grid_thw=grid.cuda(),
                        mm_token_type_ids=(ids2 == IMG).int().cuda()).logits[0, -1].float().cpu()
        _, lg2 = eng.extend(torch.tensor([nxt, 9]), return_logits=True)
        rel2 = float((lg2[0].float().cpu() - want2).abs().max() / want2.abs().max())
        assert rel2 < 3e-2, rel2
        handle.close()
    finally:
        os.environ.pop("RPU_QWEN3_5_ALLOW_ANY_PROFILE", None)
        live_handle._reset_for_tests()
