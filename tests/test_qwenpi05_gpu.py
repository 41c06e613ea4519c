"""QwenPI05 action expert (adaptive RMSNorm with a learned weight, QK norm, tanh-gated residual, SwiGLU) over an external
prefix's keys and values, against a plain fp32 PyTorch statement of the same model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _prefix(cfg, P, layers, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g) * 0.5, torch.randn(cfg.kv_heads, P, cfg.head_dim, generator=g) * 0.5)
            for _ in range(layers)]


@pytest.mark.parametrize("offset,padded,use_graph", [(0, False, True), (2, True, True), (1, True, False)])
def test_qwenpi05_action_chunk_matches_fp32(offset, padded, use_graph):
    from rhinoforge_b200.models.qwenpi05 import QwenPI05Engine, TorchQwenPI05, random_qwenpi05_state_dict, tiny_qwenpi05_config
    cfg = tiny_qwenpi05_config(prefix_layer_offset=offset)
    sd = random_qwenpi05_state_dict(cfg, seed=3, dtype=torch.float32)
    P = 37
    kv = _prefix(cfg, P, cfg.layers + offset)
    valid = torch.ones(P, dtype=torch.bool)
    if padded:
        valid[30:] = False                      # right-padded prefix: those rows are masked and do not advance positions
    g = torch.Generator().manual_seed(5)
    state = torch.randn(cfg.state_dim, generator=g)
    noise = torch.randn(cfg.horizon, cfg.action_dim, generator=g)
    eng = QwenPI05Engine(cfg, sd, max_prefix=64)
    eng.set_prefix(kv, valid)
    got = eng.predict(state, noise, use_graph=use_graph).float().cpu().clone()
    got2 = eng.predict(state, noise, use_graph=use_graph).float().cpu().clone()
    eng.check_status()
    oracle = TorchQwenPI05(cfg, sd)
    want = oracle.sample_actions(kv, valid, state, noise)
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) < 3e-2 * max(1.0, scale)
    assert torch.equal(got, got2), "a second call on the same inputs must reproduce the first bit for bit"
    # one expert pass with caller-made suffix rows and conditioning
    rows = torch.randn(cfg.suffix_rows, cfg.width, generator=g) * 0.5
    cond = torch.randn(cfg.width, generator=g) * 0.5
    h = eng.forward(rows, cond).float().cpu()
    p0 = int(valid.sum())
    ref = oracle.expert(rows, kv, valid, torch.ones(cfg.suffix_rows, dtype=torch.bool), p0 + torch.arange(cfg.suffix_rows), cond)
    assert float((h - ref).abs().max()) < 3e-2 * max(1.0, float(ref.abs().max()))
    # the prefix matters: other keys give another chunk
    eng.set_prefix(_prefix(cfg, P, cfg.layers + offset, seed=9), valid)
    other = eng.predict(state, noise, use_graph=use_graph).float().cpu()
    assert float((other - got).abs().max()) > 1e-3
    eng.close()
