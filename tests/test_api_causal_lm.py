"""RPUModelForCausalLM / RPUCache API contract: rejections before any weight is read (CPU), and
the full load -> generate path against the Hugging Face model (GPU)."""
import json
from pathlib import Path

import pytest
import torch

from test_quantization import _tiny_ckpt


@pytest.fixture()
def fresh_slot():
    from rhinoforge_b200.runtime import live_handle
    live_handle._reset_for_tests()
    yield
    live_handle._reset_for_tests()


def test_rejections_happen_before_weights_load(tmp_path, monkeypatch, fresh_slot):
    from rpu_backend import RPUModelForCausalLM
    from rpu_backend.api.errors import RPUUnsupportedDtypeError, UnsupportedModelError
    _tiny_ckpt(tmp_path / "m")
    (tmp_path / "m" / "model.safetensors").unlink()          # any weight access would now fail loudly
    load = RPUModelForCausalLM.from_pretrained
    with pytest.raises(RPUUnsupportedDtypeError):
        load(str(tmp_path / "m"), dtype=torch.float32)
    with pytest.raises(ValueError, match="reserved key"):
        load(str(tmp_path / "m"), device_map="auto")
    with pytest.raises(ValueError, match="trust_remote_code=False"):
        load(str(tmp_path / "m"), trust_remote_code=True)
    with pytest.raises(ValueError, match="positive multiple of 16"):
        load(str(tmp_path / "m"), rpu_execution={"prefill": {"chunk_size": 17}})
    with pytest.raises(ValueError, match="not supported by this model entry point"):
        load(str(tmp_path / "m"), rpu_execution={"vision": {"chunk_size": 16}})
    monkeypatch.delenv("RPU_QWEN3_ALLOW_UNLISTED_PROFILE", raising=False)
    with pytest.raises(UnsupportedModelError, match="deny by default"):
        load(str(tmp_path / "m"))                              # tiny profile is not on the allow-list
    with pytest.raises(UnsupportedModelError, match="Could not load HF config"):
        load(str(tmp_path / "missing"))
    cfg = json.loads((tmp_path / "m" / "config.json").read_text())
    cfg["architectures"] = ["Qwen3VLForConditionalGeneration"]
    (tmp_path / "m" / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(UnsupportedModelError, match="RPUModelForConditionalGeneration"):
        load(str(tmp_path / "m"))


def test_profile_tables():
    from types import SimpleNamespace as NS
    from rpu_backend.adapters.qwen3 import Qwen3Adapter
    from rpu_backend.api.errors import UnsupportedModelError
    mk = lambda h, i, l, kv, **kw: NS(hidden_size=h, intermediate_size=i, num_hidden_layers=l, num_key_value_heads=kv,
                                      num_attention_heads=h // 128, head_dim=128, **kw)
    Qwen3Adapter.preflight(mk(4096, 12288, 36, 8))
    with pytest.raises(UnsupportedModelError):
        Qwen3Adapter.preflight(mk(4096, 12288, 40, 8))
    exact = {"method": "w8a16", "quantized_lm_head": True, "lm_head_untied": True, "quantized_embed_tokens": False}
    for prof in ((5120, 17408, 40, 8), (5120, 25600, 64, 8)):
        with pytest.raises(UnsupportedModelError, match="W8A16"):
            Qwen3Adapter.preflight(mk(*prof))
        with pytest.raises(UnsupportedModelError, match="W8A16"):
            Qwen3Adapter.preflight(mk(*prof, quant_config={**exact, "quantized_embed_tokens": True}))
        Qwen3Adapter.preflight(mk(*prof, quant_config=exact))


def test_cpu_load_returns_hf_model_with_to_hook(tmp_path, monkeypatch, fresh_slot):
    from rpu_backend import RPUModelForCausalLM
    monkeypatch.setenv("RPU_QWEN3_ALLOW_UNLISTED_PROFILE", "1")
    _tiny_ckpt(tmp_path / "m")
    model = RPUModelForCausalLM.from_pretrained(str(tmp_path / "m"), rpu_execution={"prefill": {"chunk_size": 64}})
    assert type(model).__name__ == "Qwen3ForCausalLM" and next(model.parameters()).device.type == "cpu"
    assert dict(model._rpu_execution["prefill"]) == {"chunk_size": 64}
    with pytest.raises(TypeError, match="read-only"):
        model._rpu_execution["prefill"].chunk_size = 32
    assert model.to("cpu") is model


def test_cache_sizing_forms_and_position(monkeypatch):
    from types import SimpleNamespace as NS
    from rpu_backend import RPUCache
    cfg = NS(model_type="qwen3", num_hidden_layers=2, num_key_value_heads=2, num_attention_heads=4, hidden_size=256,
             head_dim=64)
    model = NS(config=cfg)
    ids = torch.zeros(1, 40, dtype=torch.long)
    with pytest.raises(ValueError, match="not both"):
        RPUCache.from_model(model, input_ids=ids, max_new_tokens=8, max_seq_len=64, device="cpu")
    with pytest.raises(ValueError, match="needs both"):
        RPUCache.from_model(model, input_ids=ids, device="cpu")
    c = RPUCache.from_model(model, input_ids=ids, max_new_tokens=8, device="cpu")
    assert c.max_seq_len >= 40 + 8 + 64 and c.max_seq_len % 16 == 0 and len(c) == 2
    c2 = RPUCache.from_model(model, max_seq_len=128, device="cpu")
    assert c2.max_seq_len == 128 and c2.position == 0
    c2.update_position(100)
    assert c2.get_seq_length() == 100 and c2.seen_tokens == 100
    with pytest.raises(ValueError, match="overflow"):
        c2.update_position(29)
    c2.reset_to_position(16)
    assert c2.position == 16
    k, v = torch.zeros(1), torch.zeros(1)
    assert c2.update(k, v, 0) == (k, v) and c2.position == 16      # HF update() is inert
    with pytest.raises(ValueError, match="float16"):
        RPUCache(2, 1, 64, 2, 64, device="cpu", dtype=torch.float32)
    with pytest.raises(ValueError, match="divisible by 16"):
        RPUCache(2, 1, 64, 2, 72, device="cpu")


def test_single_live_handle_gate(fresh_slot):
    from rhinoforge_b200.runtime import live_handle
    from rpu_backend.api.errors import RPUSingleHandleError

    class Owner:
        pass

    a, b = Owner(), Owner()
    live_handle.claim(a)
    live_handle.claim(a)                                     # idempotent for the same owner
    with pytest.raises(RPUSingleHandleError, match="already live"):
        live_handle.claim(b)
    del a
    import gc
    gc.collect()
    live_handle.claim(b)                                     # slot is free once the owner is collected
    live_handle.poison(b, "install failed")
    with pytest.raises(RPUSingleHandleError, match="process-terminal"):
        live_handle.claim(Owner())


@pytest.mark.gpu
def test_load_generate_matches_hf_model(tmp_path, monkeypatch, fresh_slot):
    from transformers import AutoModelForCausalLM
    from rpu_backend import RPUCache, RPUModelForCausalLM
    from rpu_backend.api.errors import RPUBackendError, RPUSingleHandleError
    monkeypatch.setenv("RPU_QWEN3_ALLOW_UNLISTED_PROFILE", "1")
    _tiny_ckpt(tmp_path / "m", tie=True)
    hf = AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), dtype=torch.float32).eval()
    model = RPUModelForCausalLM.from_pretrained(str(tmp_path / "m"), dtype=torch.float16, device="rpu", max_batch=2)
    with pytest.raises(RPUSingleHandleError):
        RPUModelForCausalLM.from_pretrained(str(tmp_path / "m"), device="rpu")
    with pytest.raises(RPUBackendError, match="exactly once"):
        model.to("cpu")
    ids = torch.randint(0, 512, (1, 24), generator=torch.Generator().manual_seed(0))
    cache = RPUCache.from_model(model, input_ids=ids, max_new_tokens=10)
    out = model.generate(ids, past_key_values=cache, max_new_tokens=10, do_sample=False)
    ref = hf.generate(ids, max_new_tokens=10, do_sample=False)
    assert out.shape == ref.shape and torch.equal(out[:, :24], ids)
    assert (out[:, :24 + 6] == ref[:, :24 + 6]).all()          # fp16 vs fp32: allow a late near-tie flip
    assert cache.position == 24 + 9
    # manual loop through forward(): prefill then one decode step, logits against HF
    cache2 = RPUCache.from_model(model, max_seq_len=64)
    o = model(input_ids=ids, past_key_values=cache2, logits_to_keep=1, use_cache=True, return_dict=True)
    with torch.no_grad():
        r = hf(ids).logits[:, -1]
    torch.testing.assert_close(o.logits[:, -1].float().cpu(), r, rtol=2e-2, atol=2e-2)
    assert cache2.position == 24
    dense = cache2.to_dynamic_cache()
    assert dense.get_seq_length() == 24
    model.close()


@pytest.mark.gpu
def test_hf_generate_drives_the_handle_unmodified(tmp_path, monkeypatch, fresh_slot):
    """Sampling, a stopping criterion, a left-padded batch and all-row logits go through ``GenerationMixin.generate`` /
    ``forward`` of the handle; greedy through that loop equals the handle's own graph loop."""
    from transformers import AutoModelForCausalLM, StoppingCriteria, StoppingCriteriaList
    from rpu_backend import RPUCache, RPUModelForCausalLM
    monkeypatch.setenv("RPU_QWEN3_ALLOW_UNLISTED_PROFILE", "1")
    _tiny_ckpt(tmp_path / "m", tie=True)
    hf = AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), dtype=torch.float32).eval()
    model = RPUModelForCausalLM.from_pretrained(str(tmp_path / "m"), dtype=torch.float16, device="rpu", max_batch=2)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(3, 512, (2, 12), generator=g)
    fast = model.generate(ids, past_key_values=RPUCache.from_model(model, input_ids=ids, max_new_tokens=8), max_new_tokens=8)
    slow = model.hf.generate(input_ids=ids, past_key_values=RPUCache.from_model(model, input_ids=ids, max_new_tokens=8),
                             max_new_tokens=8, do_sample=False, pad_token_id=0)
    assert torch.equal(fast.cpu(), slow.cpu())
    # sampling: deterministic under a seed, different across seeds, tokens inside the vocabulary
    outs = []
    for seed in (1, 1, 2):
        torch.manual_seed(seed)
        outs.append(model.generate(ids, max_new_tokens=8, do_sample=True, top_k=20, temperature=1.5, pad_token_id=0).cpu())
    assert torch.equal(outs[0], outs[1]) and not torch.equal(outs[0], outs[2])
    assert outs[0].shape == (2, 20) and int(outs[0].max()) < 512 and torch.equal(outs[0][:, :12], ids)

    class StopAt(StoppingCriteria):
        def __call__(self, input_ids, scores, **kw):
            return torch.full((input_ids.shape[0],), input_ids.shape[1] >= 15, dtype=torch.bool, device=input_ids.device)

    out = model.generate(ids, max_new_tokens=30, stopping_criteria=StoppingCriteriaList([StopAt()]), pad_token_id=0)
    assert out.shape[1] == 15 and torch.equal(out.cpu(), fast.cpu()[:, :15])
    # a left-padded batch equals its sequences run one by one
    short = ids[0, 5:]
    padded = torch.cat((torch.zeros(5, dtype=ids.dtype), short))[None]
    batch = torch.cat((padded, ids[1:2]))
    mask = torch.ones_like(batch)
    mask[0, :5] = 0
    both = model.generate(batch, attention_mask=mask, max_new_tokens=6, pad_token_id=0).cpu()
    alone = model.hf.generate(input_ids=short[None], past_key_values=RPUCache.from_model(model, input_ids=short[None], max_new_tokens=6),
                              max_new_tokens=6, do_sample=False, pad_token_id=0).cpu()       # the same end-of-sequence handling
    assert torch.equal(both[0, 5:], alone[0]) and torch.equal(both[1], fast.cpu()[1, :18])
    # every row's logits
    cache = RPUCache.from_model(model, max_seq_len=64, batch_size=2)
    o = model(input_ids=ids, past_key_values=cache, logits_to_keep=0)
    with torch.no_grad():
        r = hf(ids).logits
    assert o.logits.shape == r.shape
    torch.testing.assert_close(o.logits.float().cpu(), r, rtol=3e-2, atol=3e-2)
    o3 = model(input_ids=ids[:, :1] * 0 + 7, past_key_values=cache, logits_to_keep=3)       # one new token: 1 row comes back
    assert o3.logits.shape[1] == 1
    model.close()
