"""HyEmbodiedPolicy facade on the host: construction-time validation, statistics loading rules, output contract over a
fake engine and the real pre-processing, position-embedding resampling."""
import hashlib
import json
import pickle

import numpy as np
import pytest
import torch

from rhinoforge_b200.adapters.hy_vla import build_observation
from rhinoforge_b200.adapters.hy_vla.runtime import resample_pos_embedding
from rhinoforge_b200.api import HyEmbodiedPolicy, RPUBackendError, RPUConfigError, UnsupportedModelError
from rhinoforge_b200.api.hy_embodied import HyEmbodiedActionOutput, _load_norm_stats
from rhinoforge_b200.models.hyvla import LM_HEAD, assemble_prefix, random_hyvla_state_dict, tiny_hyvla_config


class _Tok:
    """Stands in for the Hugging Face tokenizer: ids by word hash, padded to max_length."""
    pad_token_id = 0

    def __call__(self, text, **kw):
        n = kw.get("max_length", 64)
        ids = [3 + (sum(map(ord, w)) % 40) for w in str(text).split()][:n]
        mask = [1] * len(ids) + [0] * (n - len(ids))
        return {"input_ids": torch.tensor([ids + [0] * (n - len(ids))]), "attention_mask": torch.tensor([mask])}


class _FakeEngine:
    dtype = torch.float16

    def __init__(self, cfg, sd, nan=False):
        self.cfg, self.sd, self.calls, self.closed, self.nan, self.last = cfg, sd, 0, False, nan, None

    def embed_images(self, images):
        return torch.ones(images.shape[0], self.cfg.grid ** 2, self.cfg.vlm_hidden)

    def build_prefix(self, embs, lang):
        return assemble_prefix(self.cfg, self.sd[LM_HEAD], embs, lang)

    def prefill(self, rows, pos, mask, vis):
        self.last = dict(S=rows.shape[0], split=int((~vis).sum()))
        return rows.shape[0]

    def denoise(self, spos, dm, state, noise, use_graph=True):
        self.calls += 1
        self.last.update(dm=tuple(dm.shape), spos0=int(spos[0]))
        out = noise.reshape(self.cfg.n_action, self.cfg.action_dim) * 0.5 + state.flatten()[0]
        return torch.full_like(out, float("nan")) if self.nan else out

    def check_status(self):
        pass

    def close(self):
        self.closed = True


def _policy(nan=False, decoder=None, **cfg_kw):
    cfg = tiny_hyvla_config(action_dim=32, state_dim=32, n_action=50, **cfg_kw)
    sd = {LM_HEAD: torch.randn(cfg.vocab, cfg.vlm_hidden)}
    eng = _FakeEngine(cfg, sd, nan)
    return HyEmbodiedPolicy._from_engine(eng, decoder=decoder, n_cameras=2), eng


def test_constructor_paths_and_argument_errors(tmp_path):
    with pytest.raises(RuntimeError, match="not a public constructor"):
        HyEmbodiedPolicy()
    with pytest.raises(UnsupportedModelError, match="w8a16"):
        HyEmbodiedPolicy.from_checkpoint(tmp_path, dtype="w8a16-expert-vlmv")
    with pytest.raises(ValueError, match="dtype must be one of"):
        HyEmbodiedPolicy.from_checkpoint(tmp_path, dtype="int3")
    for bad in (250, 8, 100):
        with pytest.raises(ValueError, match="prefix_len"):
            HyEmbodiedPolicy.from_checkpoint(tmp_path, prefix_len=bad)
    with pytest.raises(ValueError, match="not both"):
        HyEmbodiedPolicy.from_checkpoint(tmp_path, norm_stats={}, norm_stats_path="x.json")
    with pytest.raises(ValueError, match="unsupported environment key"):
        HyEmbodiedPolicy.from_checkpoint(tmp_path, runtime_env={"PATH": "/x"})
    p = HyEmbodiedPolicy.from_pretrained(tmp_path, prefix_len=192, runtime_env={"RPU_HY_VLA_UNROLL": 0})
    assert p.dtype == "fp16" and p.prefix_len == 192 and not p.action_decode_configured and p.action_dim == 20
    with pytest.raises(RPUBackendError, match=r"call \.to\('rpu'\) before infer"):
        p.infer(images=[1, 2, 3], instruction="x")
    with pytest.raises(RPUBackendError, match="accelerator only"):
        p.to("cpu")


def test_norm_stats_loading_rules(tmp_path):
    info = {"action_mean": np.zeros((50, 20)).tolist(), "action_std": np.ones((50, 20)).tolist()}
    jp = tmp_path / "norm_stats.json"
    jp.write_text(json.dumps(info))
    assert set(_load_norm_stats(str(jp), trust_pickle=False, sha256=None)) == set(info)
    pk = tmp_path / "norm_stats.pkl"
    blob = pickle.dumps(info)
    pk.write_bytes(blob)
    with pytest.raises(RPUConfigError, match="only read with trust_norm_stats_pickle"):
        _load_norm_stats(str(pk), trust_pickle=False, sha256=None)
    with pytest.raises(RPUConfigError, match="only read with trust_norm_stats_pickle"):
        _load_norm_stats(str(pk), trust_pickle=True, sha256=None)
    with pytest.raises(RPUConfigError, match="refusing to unpickle"):
        _load_norm_stats(str(pk), trust_pickle=True, sha256="0" * 64)
    assert set(_load_norm_stats(str(pk), trust_pickle=True, sha256=hashlib.sha256(blob).hexdigest())) == set(info)


def test_infer_contract_over_the_real_preprocessing():
    p, eng = _policy()
    frames = [torch.rand(3, 40, 60), torch.rand(3, 40, 60)]
    obs = build_observation(frames, "pick up the red block", _Tok(), state=np.full(20, 0.25), noise_seed=1, grid=eng.cfg.grid,
                            tokenizer_max_length=16)
    out = p.infer(obs=obs)
    assert isinstance(out, HyEmbodiedActionOutput) and out.latency_ms > 0 and set(out.phase_ms) == {"preprocess_ms", "device_ms", "decode_ms"}
    assert out.actions_full.shape == (50, 32) and out.actions_normalized.shape == (50, 20)
    assert torch.allclose(out.actions_full, obs["noise"][0] * 0.5 + 0.25)
    assert not out.physical_action_available
    with pytest.raises(RPUBackendError, match="normalized relative increments"):
        _ = out.actions
    # the prefix is cut to the real rows rounded up to 16; the suffix starts at the number of real rows
    n_valid = obs["n_valid"]
    S = (n_valid + 15) // 16 * 16
    assert eng.last["S"] == min(S, obs["prefill_pos"].numel()) and eng.last["dm"] == (51, eng.last["S"] + 51) and eng.last["spos0"] == n_valid
    with pytest.raises(ValueError, match="does not mix"):
        p.infer(obs=obs, noise_seed=3)
    with pytest.raises(ValueError, match="obs lacks"):
        p.infer(obs={k: v for k, v in obs.items() if k != "noise"})
    with pytest.raises(ValueError, match="not both"):
        p.infer(images=frames, instruction="x", ee_pose=np.zeros(16), state=np.zeros(20))
    with pytest.raises(ValueError, match="expected 2 camera images"):
        p.infer(images=frames[:1], instruction="x")
    short = HyEmbodiedPolicy._from_engine(eng, prefix_len=16, n_cameras=2)
    with pytest.raises(RPUBackendError, match="the prefix would be cut"):
        short.infer(obs=obs)
    p.close()
    p.close()
    assert eng.closed
    with pytest.raises(RPUBackendError, match="closed"):
        p.infer(obs=obs)
    pn, _ = _policy(nan=True)
    with pytest.raises(RPUBackendError, match="non-finite"):
        pn.infer(obs=obs)


def test_physical_actions_need_statistics_and_a_pose():
    from rhinoforge_b200.api.hy_action_decode import HyVlaActionDecoder
    dec = HyVlaActionDecoder.from_norm_stats_mapping({"action_mean": np.zeros((50, 20)), "action_std": np.full((50, 20), 0.01),
                                                      "qpos_mean": np.zeros(20), "qpos_std": np.ones(20)})
    p, eng = _policy(decoder=dec)
    assert p.action_decode_configured
    frames = [torch.rand(3, 40, 60), torch.rand(3, 40, 60)]
    obs = build_observation(frames, "go", _Tok(), state=np.zeros(20), noise_seed=0, grid=eng.cfg.grid, tokenizer_max_length=16)
    assert not p.infer(obs=obs).physical_action_available          # no pose in this call: nothing physical
    pose = np.array([0.3, 0.0, 0.2, 1, 0, 0, 0, 0.04, -0.3, 0.0, 0.2, 1, 0, 0, 0, 0.04])
    p._tok = _Tok()
    out = p.infer(images=frames, instruction="go", ee_pose=pose, noise_seed=0)
    assert out.physical_action_available and out.actions.shape == (49, 16) and np.isfinite(out.actions).all()
    assert p.predict_action_chunk(images=frames, instruction="go", ee_pose=pose, noise_seed=0).shape == (49, 16)


def test_position_table_resampling():
    t = torch.arange(16 * 3, dtype=torch.float32).reshape(1, 16, 3)
    assert torch.equal(resample_pos_embedding(t, 4, 4), t)
    up = resample_pos_embedding(t, 8, 8)
    assert up.shape == (1, 64, 3)
    grid4, grid8 = t[0, :, 0].reshape(4, 4), up[0, :, 0].reshape(8, 8)
    assert torch.allclose(grid8.mean(), grid4.mean(), atol=1e-4)           # bilinear, symmetric sampling keeps the mean
    assert float(grid8[0, 0]) == pytest.approx(float(grid4[0, 0]), abs=1e-5)    # border clamped
    with pytest.raises(UnsupportedModelError, match="not a square grid"):
        resample_pos_embedding(torch.zeros(1, 15, 3), 4, 4)
