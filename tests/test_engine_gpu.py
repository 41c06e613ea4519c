"""End-to-end decoder engine on the GPU against the plain-PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle_and_engine(cfg, dtype, max_batch, max_seq_len, **kw):
    from rhinoforge_b200.models.decoder import TorchDecoder, random_state_dict
    from rhinoforge_b200.runtime.engine import DecoderEngine
    sd = random_state_dict(cfg, seed=0, dtype=dtype, norm_jitter=0.05)
    oracle = TorchDecoder(cfg, sd, dtype=torch.float32, device="cuda")
    eng = DecoderEngine(cfg, lambda n: sd[n] if n in sd else sd["model.embed_tokens.weight"], dtype=dtype,
                        max_batch=max_batch, max_seq_len=max_seq_len, **kw)
    return oracle, eng


def _agree(tokens, ref_tokens, ref_logits, tol):
    """Greedy tokens must match the oracle except where the oracle's own top-2 gap is inside fp noise."""
    tokens, ref_tokens = tokens.cpu(), ref_tokens.cpu()
    B, n = ref_tokens.shape
    for b in range(B):
        for t in range(n):
            if tokens[b, t] != ref_tokens[b, t]:
                lg = ref_logits[b, t].float().cpu()
                gap = (lg[ref_tokens[b, t]] - lg[tokens[b, t]]).item()
                assert gap < tol, f"seq {b} step {t}: token {tokens[b, t]} vs oracle {ref_tokens[b, t]} (gap {gap:.4f})"
                return  # sequences legitimately diverge after a near-tie
    return


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("use_graph", [False, True])
def test_tiny_decoder_matches_oracle(dtype, use_graph):
    from rhinoforge_b200.models.decoder import tiny_config
    cfg = tiny_config()
    oracle, eng = _oracle_and_engine(cfg, dtype, max_batch=3, max_seq_len=128)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (L,), generator=g) for L in (17, 40, 5)]
    first, logits = eng.prefill(prompts, return_logits=True)
    for b, p in enumerate(prompts):
        oracle.reset()
        ref = oracle.forward(p[None].cuda())[0, -1]
        tol = 3e-2 if dtype == torch.bfloat16 else 6e-3
        torch.testing.assert_close(logits[b].float(), ref.float(), rtol=tol, atol=tol)
    toks = eng.generate(prompts, 12, use_graph=use_graph)
    for b, p in enumerate(prompts):
        rt, rl = oracle.greedy(p[None].cuda(), 12)
        _agree(toks[b:b + 1], rt, rl, 0.05 if dtype == torch.bfloat16 else 0.01)
    eng.check_status()
    eng.close()


def test_graph_replay_is_deterministic_and_matches_eager():
    from rhinoforge_b200.models.decoder import tiny_config
    cfg = tiny_config(num_layers=3)
    _, eng = _oracle_and_engine(cfg, torch.float16, max_batch=4, max_seq_len=96)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (20,), generator=g) for _ in range(4)]
    a = eng.generate(prompts, 16, use_graph=True).clone()
    b = eng.generate(prompts, 16, use_graph=True).clone()
    c = eng.generate(prompts, 16, use_graph=False).clone()
    assert torch.equal(a, b) and torch.equal(a, c)
    assert len(eng.graphs) == 1  # one BUILD, then replays only
    eng.close()


def test_chunked_prefill_equals_single_chunk():
    from rhinoforge_b200.models.decoder import tiny_config
    cfg = tiny_config()
    _, e1 = _oracle_and_engine(cfg, torch.float16, max_batch=2, max_seq_len=256, max_prefill_tokens=512)
    _, e2 = _oracle_and_engine(cfg, torch.float16, max_batch=2, max_seq_len=256, max_prefill_tokens=48)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (L,), generator=g) for L in (130, 77)]
    _, l1 = e1.prefill(prompts, return_logits=True)
    _, l2 = e2.prefill(prompts, return_logits=True)
    torch.testing.assert_close(l1.float(), l2.float(), rtol=5e-3, atol=5e-3)
    e1.close(); e2.close()


def test_gemma_style_and_gemv_decode():
    from rhinoforge_b200.models.decoder import tiny_config
    import math
    cfg = tiny_config(num_heads=4, num_kv_heads=1, head_dim=64, qk_norm=False, mlp="geglu_tanh", norm="rms_gemma",
                      embed_scale=math.sqrt(256.0), tie_embeddings=True)
    oracle, eng = _oracle_and_engine(cfg, torch.float16, max_batch=2, max_seq_len=96, decode_gemv_max_m=8)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab_size, (L,), generator=g) for L in (9, 31)]
    toks = eng.generate(prompts, 8)
    for b, p in enumerate(prompts):
        rt, rl = oracle.greedy(p[None].cuda(), 8)
        _agree(toks[b:b + 1], rt, rl, 0.02)
    eng.close()


def test_qwen3_0p6b_shape_greedy_matches_fp32_oracle():
    """Qwen3-0.6B-architecture, fp16 random init (std 0.02, seed 0), batch 1, 128 prompt ids, 32 greedy tokens."""
    from rhinoforge_b200.models.decoder import PROFILES, TorchDecoder, random_state_dict
    from rhinoforge_b200.runtime.engine import DecoderEngine
    cfg = PROFILES["qwen3-0.6b"]
    sd = random_state_dict(cfg, seed=0, std=0.02, dtype=torch.float16, device="cuda")
    eng = DecoderEngine(cfg, lambda n: sd[n] if n in sd else sd["model.embed_tokens.weight"], dtype=torch.float16,
                        max_batch=1, max_seq_len=256)
    ids = torch.randint(0, cfg.vocab_size, (128,), generator=torch.Generator().manual_seed(0))
    toks = eng.generate([ids], 32)
    oracle = TorchDecoder(cfg, sd, dtype=torch.float32, device="cuda")
    rt, rl = oracle.greedy(ids[None].cuda(), 32)
    _agree(toks, rt, rl, 0.02)
    eng.check_status()
    eng.close()


def test_causal_decoder_handle_ops_match_the_engine():
    """``torch.ops.rpu.causal_decoder_*``: create from an HF-style JSON config, install weights by name, feed input
    embeddings at position 0 and then one more row at the cached position; logits equal the engine's own."""
    import json
    from rhinoforge_b200.models.decoder import random_state_dict, tiny_config
    from rhinoforge_b200.runtime.engine import DecoderEngine
    cfg = tiny_config()
    sd = random_state_dict(cfg, seed=0, dtype=torch.float16, norm_jitter=0.05)
    get = lambda n: sd[n] if n in sd else sd["model.embed_tokens.weight"]
    eng = DecoderEngine(cfg, get, dtype=torch.float16, max_batch=2, max_seq_len=128)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (24,), generator=g) for _ in range(2)]
    _, want = eng.prefill(prompts, return_logits=True)
    nxt = [torch.randint(0, cfg.vocab_size, (1,), generator=g) for _ in range(2)]
    _, want2 = eng.extend(nxt, return_logits=True)
    want, want2 = want.clone(), want2.clone()
    eng.close()

    hf = dict(model_type="qwen3", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
              intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_layers, num_attention_heads=cfg.num_heads,
              num_key_value_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_eps, rope_theta=cfg.rope_theta,
              tie_word_embeddings=cfg.tie_embeddings, max_position_embeddings=cfg.max_position, rpu_max_batch=2,
              rpu_max_seq_len=128)
    ops = torch.ops.rpu
    h = ops.causal_decoder_create(json.dumps(hf))
    names = list(sd)
    if "lm_head.weight" not in sd:
        names.append("lm_head.weight")
    ops.causal_decoder_set_weights(h, names, [get(n) for n in names])
    emb = sd["model.embed_tokens.weight"].cuda()
    x = torch.stack([emb[p.cuda()] for p in prompts])
    got = ops.causal_decoder_forward(h, x, [], [], None, 0, True, None, None, None, None)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-3, atol=2e-3)
    x2 = torch.stack([emb[p.cuda()] for p in nxt])
    got2 = ops.causal_decoder_forward(h, x2, [], [], None, 24, True, None, None, None, None)
    torch.testing.assert_close(got2.float(), want2.float(), rtol=2e-3, atol=2e-3)
    with pytest.raises(Exception, match="does not match the cached lengths"):
        ops.causal_decoder_forward(h, x2, [], [], None, 7, True, None, None, None, None)
    ops.causal_decoder_destroy(h)


def test_engine_over_an_interleaved_oversubscribed_page_table():
    """KV pages are handed out on demand: three sequences that grow in turns end up with interleaved page ids in a
    pool smaller than ``batch * max_seq_len``; greedy tokens still follow the fp32 oracle, and a request the pool
    cannot hold is refused on the host before anything runs."""
    from rhinoforge_b200.api.errors import SPMExhaustionError
    from rhinoforge_b200.models.decoder import tiny_config
    cfg = tiny_config()
    oracle, eng = _oracle_and_engine(cfg, torch.float16, max_batch=3, max_seq_len=256, kv_pool_tokens=3 * 96)
    assert eng.cache.num_pages == 18 < 3 * eng.cache.pages_per_seq
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab_size, (L,), generator=g) for L in (17, 40, 5)]
    first = eng.prefill(prompts)
    parts = [first[:, None]]
    for _ in range(4):                       # four decode calls of 9 steps: every call adds pages to some sequence
        parts.append(eng.decode(9).clone())
    toks = torch.cat(parts, 1)
    table = eng.cache._pt_host[:, :8].tolist()
    owned = [eng.cache.owned_pages(s) for s in range(3)]
    assert owned == [(17 + 36 + 1 + 15) // 16, (40 + 36 + 1 + 15) // 16, (5 + 36 + 1 + 15) // 16]
    rows = [table[s][:owned[s]] for s in range(3)]
    assert any(r != list(range(r[0], r[0] + len(r))) for r in rows), rows      # not the identity / contiguous map
    assert len({p for r in rows for p in r}) == sum(owned)                       # no page is shared
    for b, p in enumerate(prompts):
        rt, rl = oracle.greedy(p[None].cuda(), 37)
        _agree(toks[b:b + 1], rt, rl, 0.01)
    eng.check_status()
    free = eng.cache.free_pages()
    with pytest.raises(SPMExhaustionError):
        eng.decode(40)                        # 6 + 8 + 6 pages would be needed, the pool has 18
    assert eng.cache.free_pages() <= free
    eng.close()
