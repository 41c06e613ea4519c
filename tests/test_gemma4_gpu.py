"""Head-size-512 attention and the Gemma4 text decoder against PyTorch / Hugging Face fp32."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _sdpa_ref(q, k, v, qlen, kvlen, Hq, Hkv, hd, causal, window, scale):
    """q [qlen, Hq*hd], k/v [kvlen, Hkv*hd] fp32 -> [qlen, Hq*hd]; query i sits at position kvlen - qlen + i."""
    qh = q.view(qlen, Hq, hd).transpose(0, 1)
    kh = k.view(kvlen, Hkv, hd).transpose(0, 1).repeat_interleave(Hq // Hkv, 0)
    vh = v.view(kvlen, Hkv, hd).transpose(0, 1).repeat_interleave(Hq // Hkv, 0)
    s = qh @ kh.transpose(1, 2) * scale
    qp = torch.arange(qlen, device=q.device)[:, None] + (kvlen - qlen)
    kp = torch.arange(kvlen, device=q.device)[None, :]
    ok = torch.ones(qlen, kvlen, dtype=torch.bool, device=q.device)
    if causal:
        ok &= kp <= qp
    if window > 0:
        ok &= kp > qp - window
    s = s.masked_fill(~ok, float("-inf"))
    return (torch.softmax(s, -1) @ vh).transpose(0, 1).reshape(qlen, Hq * hd)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal,window", [(True, 0), (True, 24), (False, 0)])
def test_attention_head_dim_512(dtype, causal, window):
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(0)
    Hq, Hkv, hd = 4, 2, 512
    qlens, kvlens = [70, 1, 33], [70, 91, 50]                  # prefill, decode over a context, a continuation
    Tq, rows = sum(qlens), 128
    q = (torch.randn(Tq, Hq * hd, device="cuda") * 0.3).to(dtype)
    kc = (torch.randn(3 * rows, Hkv * hd, device="cuda") * 0.3).to(dtype)
    vc = torch.randn(3 * rows, Hkv * hd, device="cuda").to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    q_start = i32([0, 70, 71])
    out = torch.zeros(Tq, Hq * hd, device="cuda", dtype=dtype)
    scale = 1.0 / math.sqrt(hd) if window == 0 else 0.08
    K.attention_prefill(q, out, Hq=Hq, Hkv=Hkv, hd=hd, q_start=q_start, q_len=i32(qlens), kv_len=i32(kvlens), max_q_len=max(qlens),
                        k=kc, v=vc, kv_start=i32([0, rows, 2 * rows]), causal=causal, window=window, scale=scale)
    torch.cuda.synchronize()
    o = 0
    for s, (ql, kl) in enumerate(zip(qlens, kvlens)):
        ref = _sdpa_ref(q[o:o + ql].float(), kc[s * rows:s * rows + kl].float(), vc[s * rows:s * rows + kl].float(), ql, kl, Hq, Hkv, hd,
                        causal, window, scale)
        err = float((out[o:o + ql].float() - ref).abs().max())
        assert err < (6e-3 if dtype == torch.float16 else 4e-2), (s, err)
        o += ql


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("causal,window", [(True, 0), (True, 9), (False, 0)])
def test_attention_short_problem_route(hd, causal, window):
    """At most 64 query rows over at most 512 keys with a host-side key bound: the register-accumulator kernel takes heads of
    64 / 128 too; its result against fp32, and the launch goes to that kernel (its name in the launch tally)."""
    from rhinoforge_b200.ops import kernels as K
    torch.manual_seed(1)
    dtype = torch.float16
    Hq, Hkv = 6, 3
    qlens, kvlens = [24, 1, 41, 64], [24, 34, 300, 64]
    Tq, rows = sum(qlens), 320
    q = (torch.randn(Tq, Hq * hd, device="cuda") * 0.4).to(dtype)
    kc = (torch.randn(4 * rows, Hkv * hd, device="cuda") * 0.4).to(dtype)
    vc = torch.randn(4 * rows, Hkv * hd, device="cuda").to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    q_start = i32([0, 24, 25, 66])
    scale = 1.0 / math.sqrt(hd)
    outs = []
    for bound in (300, 0):                                       # 0: bound unknown, the tensor-memory kernel runs
        out = torch.zeros(Tq, Hq * hd, device="cuda", dtype=dtype)
        K.attention_prefill(q, out, Hq=Hq, Hkv=Hkv, hd=hd, q_start=q_start, q_len=i32(qlens), kv_len=i32(kvlens), max_q_len=max(qlens),
                            k=kc, v=vc, kv_start=i32([0, rows, 2 * rows, 3 * rows]), causal=causal, window=window, scale=scale,
                            max_kv_len=bound)
        torch.cuda.synchronize()
        outs.append(out)
    o = 0
    for s, (ql, kl) in enumerate(zip(qlens, kvlens)):
        ref = _sdpa_ref(q[o:o + ql].float(), kc[s * rows:s * rows + kl].float(), vc[s * rows:s * rows + kl].float(), ql, kl, Hq, Hkv, hd,
                        causal, window, scale)
        for out in outs:
            err = float((out[o:o + ql].float() - ref).abs().max())
            assert err < 6e-3, (s, err)
        o += ql


def _tiny_gemma4(**over):
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig
    from transformers.models.gemma4.modeling_gemma4 import Gemma4ForCausalLM
    kw = dict(vocab_size=300, hidden_size=128, intermediate_size=256, num_hidden_layers=6, num_attention_heads=2,
              num_key_value_heads=1, head_dim=256, global_head_dim=512, sliding_window=16,
              layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2, num_kv_shared_layers=2,
              hidden_size_per_layer_input=32, vocab_size_per_layer_input=300, max_position_embeddings=256,
              rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                               "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1000000.0}},
              tie_word_embeddings=True, pad_token_id=0)
    kw.update(over)
    c = Gemma4TextConfig(**kw)
    c._attn_implementation = "eager"
    torch.manual_seed(0)
    m = Gemma4ForCausalLM(c).float().eval()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * (0.5 if "embed" in n else 0.06))
            else:
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
        for i, layer in enumerate(m.model.layers):
            layer.layer_scalar.fill_(0.8 + 0.05 * i)
    return c, m


@pytest.mark.parametrize("over", [{}, {"num_kv_shared_layers": 0, "hidden_size_per_layer_input": 0, "final_logit_softcapping": 30.0}])
def test_gemma4_engine_matches_hf(over):
    from rhinoforge_b200.models.gemma4 import Gemma4Engine
    c, ref = _tiny_gemma4(**over)
    sd = ref.state_dict()
    eng = Gemma4Engine(c, lambda n: sd[n], max_seq_len=128, max_batch=2, max_tokens=128, dtype=torch.float16)
    g = torch.Generator().manual_seed(3)
    a, b = torch.randint(1, 300, (41,), generator=g), torch.randint(1, 300, (23,), generator=g)
    got = eng.prefill([a, b], all_logits=True)
    eng.check_status()
    for ids, lg in zip((a, b), got):
        with torch.no_grad():
            want = ref(ids[None]).logits[0]
        err = float((lg.cpu() - want).abs().max() / want.abs().max())
        assert err < 4e-2, err
    # greedy decode of both sequences against Hugging Face run one by one
    steps = 6
    eng.reset()
    toks = eng.generate([a, b], steps).cpu()
    for r, ids in enumerate((a, b)):
        with torch.no_grad():
            want = ref.generate(ids[None], max_new_tokens=steps, do_sample=False)[0, ids.numel():]
        agree = int((toks[r, :want.numel()] == want).sum())
        assert toks[r, 0] == want[0] and agree >= steps - 1, (toks[r].tolist(), want.tolist())
    # the graph replay equals the eager step
    eng.reset()
    first = eng.prefill([a, b]).argmax(-1).to(torch.int32)
    eager = eng.decode(first, 3, use_graph=False).cpu()
    assert torch.equal(eager, toks[:, 1:4])
    eng.close()


def test_gemma4_e4b_widths_reduced_depth():
    """E4B layer geometry at its real widths (hidden 2560, 8 / 2 heads of 256 and 512, window 512, PLE 256) on six layers
    and a small vocabulary: a 700-token prompt (longer than the window) and a batch-2 decode against Hugging Face fp32."""
    from rhinoforge_b200.models.gemma4 import Gemma4Engine
    c, ref = _tiny_gemma4(vocab_size=2048, vocab_size_per_layer_input=2048, hidden_size=2560, intermediate_size=10240,
                          num_attention_heads=8, num_key_value_heads=2, sliding_window=512, hidden_size_per_layer_input=256,
                          max_position_embeddings=2048,
                          layer_types=["sliding_attention"] * 2 + ["full_attention"] + ["sliding_attention"] * 2 + ["full_attention"])
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if p.dim() >= 2 and "embed" not in n:
                p.mul_(0.35)                                   # keep activations in range at this width
    ref = ref.cuda()
    sd = ref.state_dict()
    eng = Gemma4Engine(c, lambda n: sd[n], max_seq_len=1024, max_batch=2, max_tokens=1024, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(7)
    a, b = torch.randint(1, 2048, (700,), generator=g), torch.randint(1, 2048, (150,), generator=g)
    got = eng.prefill([a, b])
    eng.check_status()
    for r, ids in enumerate((a, b)):
        with torch.no_grad():
            want = ref(ids[None].cuda()).logits[0, -1].float()
        err = float((got[r] - want).abs().max() / want.abs().max())
        assert err < 8e-2, (r, err)
    first = got.argmax(-1).to(torch.int32)
    toks = eng.decode(first, 4)
    eng.check_status()
    assert toks.shape == (2, 4) and int(toks.max()) < 2048
    eng.close()


def test_gemma4_adapter_handle():
    from rhinoforge_b200.adapters.gemma4 import Gemma4Adapter
    c, ref = _tiny_gemma4()
    handle = Gemma4Adapter(ref, dtype=torch.float16).to_rpu(max_seq_len=96, max_batch=2)
    ids = torch.randint(1, 300, (2, 20), generator=torch.Generator().manual_seed(4))
    out = handle(ids)
    with torch.no_grad():
        want = ref(ids).logits
    assert out.logits.shape == want.shape
    assert float((out.logits.cpu() - want).abs().max() / want.abs().max()) < 4e-2
    gen = handle.generate(ids, max_new_tokens=4)
    assert gen.shape == (2, 24) and torch.equal(gen[:, :20], ids)
    with torch.no_grad():
        hf = ref.generate(ids, max_new_tokens=4, do_sample=False)
    assert torch.equal(gen[:, 20], hf[:, 20])
    handle.close()
