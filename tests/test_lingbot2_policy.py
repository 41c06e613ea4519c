"""Lingbot2Policy facade on the host: construction-time validation, lifecycle, output contract (fake engine)."""
import json

import pytest
import torch

from rhinoforge_b200.api import Lingbot2Policy, RPUBackendError, UnsupportedModelError
from rhinoforge_b200.api.lingbot2 import VALID_ACTION_DIMS, Lingbot2ActionOutput


class _FakeVlm:
    class vcfg:
        spatial_merge_size = 2


class _FakeEngine:
    """Stands in for Lingbot2Engine: deterministic output from the inputs, counts calls."""
    dtype = torch.float16
    max_prefix = 64
    _graphs = {10: object()}

    def __init__(self, nan=False):
        from rhinoforge_b200.models.lingbot2 import Lingbot2Config
        self.cfg, self.vlm, self.calls, self.closed, self.nan = Lingbot2Config(), _FakeVlm(), 0, False, nan

    def build_input_ids(self, per_image, lang):
        return torch.cat([torch.full((n,), 150) for n in per_image] + [lang.flatten()])

    def predict(self, ids, px, grid, state, noise, use_graph=True):
        self.calls += 1
        out = noise * 0.5 + state[:1]
        return torch.full_like(out, float("nan")) if self.nan else out

    def check_status(self):
        pass

    def close(self):
        self.closed = True


def _obs():
    return {"pixel_values": torch.zeros(48, 1536), "image_grid_thw": torch.tensor([[1, 4, 6], [1, 4, 6]]),
            "lang_tokens": torch.tensor([3, 4, 5]), "state": torch.arange(55.0), "noise": torch.ones(50, 55)}


def test_constructor_paths_and_argument_errors(tmp_path):
    with pytest.raises(RuntimeError, match="not a public constructor"):
        Lingbot2Policy()
    with pytest.raises(UnsupportedModelError, match="w8a16"):
        Lingbot2Policy.from_checkpoint(tmp_path, dtype="w8a16")
    with pytest.raises(ValueError, match="dtype must be one of"):
        Lingbot2Policy.from_checkpoint(tmp_path, dtype="int3")
    with pytest.raises(ValueError, match="max_lang_tokens"):
        Lingbot2Policy.from_checkpoint(tmp_path, max_lang_tokens=0)
    with pytest.raises(ValueError, match="unsupported environment key"):
        Lingbot2Policy.from_checkpoint(tmp_path, runtime_env={"PATH": "/x"})
    p = Lingbot2Policy.from_checkpoint(tmp_path, runtime_env={"RPU_LINGBOT2_DENOISE_UNROLL": 1})
    assert p.dtype == "fp16" and not p.robot_ready and not p.graphs_ready and p.graph_profile is None
    with pytest.raises(RPUBackendError, match=r"call \.to\('rpu'\) before infer"):
        p.infer(obs=_obs())
    with pytest.raises(RPUBackendError, match="accelerator only"):
        p.to("cpu")


def test_infer_output_contract_and_lifecycle():
    eng = _FakeEngine()
    p = Lingbot2Policy._from_engine(eng)
    out = p.infer(obs=_obs())
    assert isinstance(out, Lingbot2ActionOutput) and out.latency_ms > 0.0
    assert out.actions_full.shape == (50, 55) and out.actions_normalized.shape == (50, VALID_ACTION_DIMS)
    assert torch.allclose(out.actions_full, torch.full((50, 55), 0.5))
    assert not out.robot_ready and out.extra["denormalized"] is False and out.extra["graphs_ready"] is False
    with pytest.raises(RPUBackendError, match="normalized, not physical-unit"):
        _ = out.actions
    with pytest.raises(ValueError, match="pass either obs"):
        p.infer(images=[1])
    p.prepare_graphs(obs=_obs())                      # BUILD + REPLAY + determinism check + freeze
    assert eng.calls == 3 and p.graphs_ready and p.graph_profile["deterministic"] and p.graph_profile["num_steps"] == 10
    with pytest.raises(RuntimeError, match="already prepared"):
        p.prepare_graphs(obs=_obs())
    assert p.infer(obs=_obs()).extra["graphs_ready"] is True
    p.close()
    assert eng.closed and not p.graphs_ready
    with pytest.raises(RPUBackendError, match="closed"):
        p.infer(obs=_obs())
    p.close()                                          # idempotent


def test_non_finite_actions_are_refused_and_denormalisation_is_applied(tmp_path):
    with pytest.raises(RPUBackendError, match="non-finite action chunk"):
        Lingbot2Policy._from_engine(_FakeEngine(nan=True)).infer(obs=_obs())
    from rhinoforge_b200.api.action_denorm import ActionDenormalizer, ActionGroup
    stats = {"norm_stats": {"action.arm": {"mean": [1.0] * 14, "std": [2.0] * 14}, "action.grip": {"min": [0.0] * 2, "max": [0.1] * 2}}}
    path = tmp_path / "norm.json"
    path.write_text(json.dumps(stats))
    d = ActionDenormalizer.from_spec(str(path), [ActionGroup("action.arm", 14, "meanstd"), ActionGroup("action.grip", 2, "minmax")])
    out = Lingbot2Policy._from_engine(_FakeEngine(), denorm=d).infer(obs=_obs())
    assert out.robot_ready and out.actions.shape == (50, 16)
    assert torch.allclose(out.actions[:, :14], torch.full((50, 14), 0.5 * (2.0 + 1e-6) + 1.0), atol=1e-5)
    assert torch.allclose(out.actions[:, 14:], torch.full((50, 2), (0.5 + 1) / 2 * (0.1 + 1e-6)), atol=1e-5)


def test_adapter_preflight_reads_geometry_from_the_checkpoint_config():
    from rhinoforge_b200.adapters.lingbot_vla_v2 import expert_config
    cfg = expert_config({"expert_hidden_size": 768, "num_experts": 32, "num_experts_per_tok": 4, "chunk_size": 50,
                         "max_action_dim": 55, "expert": {"moe_intermediate_size": 512}}, 5e6)
    assert (cfg.hidden, cfg.experts, cfg.top_k, cfg.horizon, cfg.action_dim, cfg.routed_inter) == (768, 32, 4, 50, 55, 512)
    with pytest.raises(UnsupportedModelError, match="head_dim 96"):
        expert_config({"expert_head_dim": 96}, 1e6)
    with pytest.raises(UnsupportedModelError, match="top-9 of 8"):
        expert_config({"num_experts": 8, "num_experts_per_tok": 9}, 1e6)
