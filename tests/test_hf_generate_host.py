"""Hugging Face ``generate()`` driving the handle's ``forward`` unmodified: plumbing checked on the CPU with a stand-in
handle whose ``forward`` is a tiny Hugging Face model behind the same contract (drops padding, one row per step)."""
import pytest
import torch

from rhinoforge_b200.runtime.hf_generation import make_adapter


def _tiny():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                      vocab_size=50, max_position_embeddings=128, pad_token_id=0, eos_token_id=49, bos_token_id=1)
    torch.manual_seed(0)
    return cfg, LlamaForCausalLM(cfg).float().eval()


class _FakeCache:
    """Stands in for the accelerator cache: remembers the real tokens seen per sequence."""

    is_compileable = False

    def __init__(self):
        self.tokens = None

    @property
    def position(self):
        return 0 if self.tokens is None else max(len(t) for t in self.tokens)

    def get_seq_length(self, layer_idx=0):
        return self.position


class _FakeHandle:
    """``forward`` with the handle's contract, computed by re-running the tiny model on each sequence's real tokens."""

    def __init__(self, cfg, model):
        self.config, self.model, self.device, self.dtype = cfg, model, torch.device("cpu"), torch.float32
        self.generation_config = None
        self.calls = []

    def forward(self, input_ids, past_key_values, attention_mask=None, logits_to_keep=1, use_cache=True, return_dict=True):
        from rhinoforge_b200.runtime.causal_lm import RPUCausalLM
        from transformers.modeling_outputs import CausalLMOutputWithPast
        rows, _ = RPUCausalLM._unpad(input_ids, attention_mask)
        self.calls.append((tuple(int(r.numel()) for r in rows), int(logits_to_keep)))
        c = past_key_values
        if c.tokens is None:
            c.tokens = [[] for _ in rows]
        out = []
        for b, r in enumerate(rows):
            c.tokens[b].extend(r.tolist())
            with torch.no_grad():
                lg = self.model(torch.tensor([c.tokens[b]])).logits[0]
            out.append(lg[-1:])
        assert logits_to_keep == 1
        return CausalLMOutputWithPast(logits=torch.stack(out), past_key_values=c)


def test_sampling_through_hf_generate_matches_the_model_itself():
    cfg, model = _tiny()
    h = _FakeHandle(cfg, model)
    ad = make_adapter(h)
    ids = torch.tensor([[1, 5, 9, 13], [1, 7, 3, 21]])
    torch.manual_seed(123)
    want = model.generate(ids, do_sample=True, top_k=8, temperature=0.9, max_new_tokens=12, pad_token_id=0)
    torch.manual_seed(123)
    got = ad.generate(input_ids=ids, past_key_values=_FakeCache(), do_sample=True, top_k=8, temperature=0.9, max_new_tokens=12,
                      pad_token_id=0)
    assert torch.equal(got, want)
    assert h.calls[0] == ((4, 4), 1) and all(c == ((1, 1), 1) for c in h.calls[1:])


def test_left_padded_batch_and_stopping_criteria():
    from transformers import StoppingCriteria, StoppingCriteriaList
    cfg, model = _tiny()
    h = _FakeHandle(cfg, model)
    ad = make_adapter(h)
    ids = torch.tensor([[0, 0, 1, 5, 9], [1, 7, 3, 21, 8]])
    mask = torch.tensor([[0, 0, 1, 1, 1], [1, 1, 1, 1, 1]])
    want = model.generate(ids, attention_mask=mask, do_sample=False, max_new_tokens=9, pad_token_id=0)
    got = ad.generate(input_ids=ids, attention_mask=mask, past_key_values=_FakeCache(), do_sample=False, max_new_tokens=9, pad_token_id=0)
    assert torch.equal(got, want)
    assert h.calls[0] == ((3, 5), 1)

    class StopAfter(StoppingCriteria):
        def __call__(self, input_ids, scores, **kw):
            return torch.full((input_ids.shape[0],), input_ids.shape[1] >= 8, dtype=torch.bool)

    got = ad.generate(input_ids=ids, attention_mask=mask, past_key_values=_FakeCache(), do_sample=False, max_new_tokens=20,
                      pad_token_id=0, stopping_criteria=StoppingCriteriaList([StopAfter()]))
    assert got.shape[1] == 8 and torch.equal(got, want[:, :8])


def test_handle_routes_plain_greedy_to_the_fast_path_and_the_rest_to_hf():
    from rhinoforge_b200.runtime.causal_lm import RPUCausalLM
    seen = {}

    class Eng:
        device, dtype = torch.device("cpu"), torch.float32

        def check_status(self):
            seen["checked"] = True

    class Hf:
        def generate(self, **kw):
            seen["hf"] = kw
            return kw["input_ids"]

    m = object.__new__(RPUCausalLM)
    m.engine, m._hf_adapter = Eng(), Hf()
    ids = torch.tensor([[1, 2, 3]])
    cache = object()
    out = m.generate(ids, past_key_values=cache, max_new_tokens=4, do_sample=True, top_p=0.9)
    assert out is ids and seen["hf"]["do_sample"] is True and seen["hf"]["top_p"] == 0.9 and seen["hf"]["max_new_tokens"] == 4
    assert seen["hf"]["past_key_values"] is cache and seen["checked"]
    seen.clear()
    m.generate(ids, past_key_values=cache, max_new_tokens=4, attention_mask=torch.tensor([[0, 1, 1]]))
    assert "hf" in seen                                        # a padded batch is Hugging Face's loop too
    seen.clear()
    m.generate(ids, past_key_values=cache, max_length=9)
    assert seen["hf"]["max_length"] == 9


def test_unpad_rejects_holes_and_tracks_running_masks():
    from rhinoforge_b200.runtime.causal_lm import RPUCausalLM
    from rhinoforge_b200.runtime.errors import RPUBackendError
    ids = torch.tensor([[4, 5, 6], [7, 8, 9]])
    rows, keep = RPUCausalLM._unpad(ids, torch.tensor([[0, 1, 1], [1, 1, 1]]))
    assert rows[0].tolist() == [5, 6] and rows[1].tolist() == [7, 8, 9] and keep[0].tolist() == [1, 2]
    with pytest.raises(RPUBackendError, match="holes"):
        RPUCausalLM._unpad(ids, torch.tensor([[1, 0, 1], [1, 1, 1]]))
    # decode step: the mask covers prompt + generated columns, the input is the last column
    rows, keep = RPUCausalLM._unpad(ids[:, -1:], torch.tensor([[0, 1, 1, 1], [1, 1, 1, 1]]))
    assert keep is None and [r.tolist() for r in rows] == [[6], [9]]
