"""Hy-Embodied VLA towers (row-routed twin weights, RoPE before the shared per-head norm, expert over the shared cache)
against a plain fp32 PyTorch statement that selects the weight set row by row."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(cfg, seed=0, n_img=2, n_lang=5, pad=3):
    from rhinoforge_b200.models.hyvla import LM_HEAD, assemble_prefix
    g = torch.Generator().manual_seed(seed)
    return g


@pytest.mark.parametrize("use_graph", [True, False])
def test_hyvla_prefill_and_action_chunk_match_fp32(use_graph):
    from rhinoforge_b200.models.hyvla import (LM_HEAD, HyVlaEngine, TorchHyVla, assemble_prefix, random_hyvla_state_dict,
                                              tiny_hyvla_config)
    cfg = tiny_hyvla_config()
    sd = random_hyvla_state_dict(cfg, seed=3)
    g = torch.Generator().manual_seed(5)
    imgs = [torch.randn(cfg.grid ** 2, cfg.vlm_hidden, generator=g) * 0.5 for _ in range(2)]
    lang = torch.randint(0, 50, (5,), generator=g)
    rows, vis = assemble_prefix(cfg, sd[LM_HEAD], imgs, lang)
    S = rows.shape[0]
    valid = torch.ones(S, dtype=torch.bool)
    valid[-2:] = False                                      # two padded language rows at the end
    pos = (torch.cumsum(valid.long(), 0) - 1).clamp_min(0)
    mask = torch.tril(torch.ones(S, S, dtype=torch.bool)) & valid[None] & valid[:, None]
    L = cfg.suffix_len
    dm = torch.zeros(L, S + L, dtype=torch.bool)
    dm[:, :S] = valid[None]
    dm[0, S] = True                                         # the state row sees itself
    dm[1:, S:] = True                                       # action rows see the whole suffix
    spos = int(valid.sum()) + torch.arange(L)
    state = torch.randn(cfg.state_dim, generator=g)
    noise = torch.randn(cfg.n_action, cfg.action_dim, generator=g)
    eng = HyVlaEngine(cfg, sd, max_prefix=64)
    assert eng.prefill(rows, pos, mask, vis) == S
    oracle = TorchHyVla(cfg, sd)
    kv = oracle.prefill(rows, pos, mask, vis)
    for i in (0, cfg.layers - 1):                           # cache rows are in the prefix's own order
        k, v = eng.cache.gather(i, 0, S)
        wk, wv = kv[i][0].transpose(0, 1), kv[i][1].transpose(0, 1)
        assert float((k.float().cpu()[:, valid] - wk[:, valid]).abs().max()) < 3e-2 * max(1.0, float(wk.abs().max()))
        assert float((v.float().cpu()[:, valid] - wv[:, valid]).abs().max()) < 3e-2 * max(1.0, float(wv.abs().max()))
    got = eng.denoise(spos, dm, state, noise, use_graph=use_graph).float().cpu().clone()
    got2 = eng.denoise(spos, dm, state, noise, use_graph=use_graph).float().cpu().clone()
    eng.check_status()
    want = oracle.sample_actions(kv, spos, dm, state, noise)
    assert float((got - want).abs().max()) < 3e-2 * max(1.0, float(want.abs().max()))
    assert torch.equal(got, got2)
    # routing matters: with every row sent through the text weights the keys differ
    kv_text = oracle.prefill(rows, pos, mask, torch.zeros_like(vis))
    assert float((kv_text[1][0] - kv[1][0]).abs().max()) > 1e-3
    eng.close()
