"""Wall-OSS on the host: facade validation and output contract (fake engine), prompt text, state string, normaliser,
action mask, masked-DOF blend inputs, preprocessor fold, checkpoint-name translation."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from rhinoforge_b200.adapters.wall_oss import (Normalizer, action_config, build_flow_prompt, discretize_proprioception,
                                               expand_image_tokens, text_config)
from rhinoforge_b200.api import RPUBackendError, UnsupportedModelError, WallOssPolicy
from rhinoforge_b200.api.wall_oss import WallOssActionOutput
from rhinoforge_b200.models.wall_oss import (PRE_P, VisionNames, action_mask, expert0_getter, flow_times, folded_preprocessor,
                                             masked_dof_inputs, random_wall_oss_expert, sinusoidal_pos_emb,
                                             tiny_wall_oss_config, wall_oss_expert_shapes)


class _FakeEngine:
    dtype = torch.float16
    max_prefix, max_seq = 64, 80
    _graphs = {(10, False): object()}

    def __init__(self, nan=False):
        self.cfg, self.calls, self.closed, self.nan, self.last = tiny_wall_oss_config(num_steps=10), 0, False, nan, None

    def predict(self, ids, px, grid, noise, dof, num_steps, *, padding_action=None, use_graph=True):
        self.calls += 1
        self.last = dict(num_steps=num_steps, padding=padding_action, use_graph=use_graph)
        out = noise * 0.5 * dof + (0 if padding_action is None else padding_action * (1 - dof))
        return torch.full_like(out, float("nan")) if self.nan else out

    def check_status(self):
        pass

    def close(self):
        self.closed = True


def _norm(ad=6, pd=4):
    a = {"min.robot": torch.full((ad,), -2.0), "delta.robot": torch.full((ad,), 4.0)}
    p = {"min.robot": torch.full((pd,), -1.0), "delta.robot": torch.full((pd,), 2.0)}
    return Normalizer(a, p, "robot")


def _obs():
    return {"input_ids": torch.arange(12), "pixel_values": None, "image_grid_thw": None}


def test_constructor_paths_and_argument_errors(tmp_path):
    with pytest.raises(RuntimeError, match="not a public constructor"):
        WallOssPolicy()
    for flag in ("w8a16", "w4a16", "nvfp4a16"):
        with pytest.raises(UnsupportedModelError, match="16 bits"):
            WallOssPolicy.from_checkpoint(tmp_path, **{flag: True})
    with pytest.raises(ValueError, match="mutually exclusive"):
        WallOssPolicy.from_checkpoint(tmp_path, w8a16=True, w4a16=True)
    with pytest.raises(UnsupportedModelError, match="rtc=True"):
        WallOssPolicy.from_checkpoint(tmp_path, rtc=True)
    with pytest.raises(ValueError, match="camera_names"):
        WallOssPolicy.from_checkpoint(tmp_path, camera_names=("periscope",))
    with pytest.raises(ValueError, match="state_bins"):
        WallOssPolicy.from_checkpoint(tmp_path, state_bins=1)
    with pytest.raises(ValueError, match="max_seq_len"):
        WallOssPolicy.from_checkpoint(tmp_path, max_seq_len=40, action_horizon=32)
    with pytest.raises(ValueError, match="active_slots"):
        WallOssPolicy.from_checkpoint(tmp_path, active_slots=[1, 1])
    with pytest.raises(ValueError, match="unsupported environment key"):
        WallOssPolicy.from_checkpoint(tmp_path, runtime_env={"PATH": "/x"})
    with pytest.raises(ValueError, match="not supported by this model entry point|unknown stage"):
        WallOssPolicy.from_checkpoint(tmp_path, rpu_execution={"denoise": {"chunk_size": 16}})
    p = WallOssPolicy.from_pretrained(tmp_path, runtime_env={"RPU_WALL_OSS_FUSED_DENOISE": 0}, camera_names=["face_view", "top_view"])
    assert p.precision == "fp16" and p.camera_names == ["face_view", "top_view"] and p.action_horizon == 32
    assert not p.graphs_ready and p.graph_profile is None
    with pytest.raises(RPUBackendError, match="complete live runtime before inference"):
        p.infer(obs=_obs())
    with pytest.raises(RPUBackendError, match="accelerator only"):
        p.to("cpu")


def test_infer_output_contract_masks_and_lifecycle():
    eng = _FakeEngine()
    p = WallOssPolicy._from_engine(eng, normalizer=_norm())
    H, AD = eng.cfg.horizon, eng.cfg.action_dim
    out = p.infer(obs=_obs(), noise=torch.ones(H, AD))
    assert isinstance(out, WallOssActionOutput) and out.latency_ms > 0.0 and out.action_hz == 32.0
    assert out.actions.shape == (H, AD) and out.actions.dtype == torch.float32
    assert torch.allclose(out.extra["x_norm"], torch.full((H, AD), 0.5))
    assert torch.allclose(out.actions, torch.full((H, AD), (0.5 + 1) / 2 * 4.0 - 2.0))       # (x + 1) / 2 * delta + min
    assert set(out.phase_ms) == {"preprocess_ms", "device_ms", "postprocess_ms"} and out.extra["prefix_len"] == 12
    assert eng.last["padding"] is None and eng.last["use_graph"] is True
    # a seeded default noise is reproducible and differs by seed
    a, b, c = (p.infer(obs=_obs(), noise_seed=s).extra["x_norm"] for s in (0, 0, 1))
    assert torch.equal(a, b) and not torch.equal(a, c)
    # inactive degrees of freedom end on normalised physical zero: 2 * (0 - min) / delta - 1 = 0
    dof = torch.ones(H, AD)
    dof[:, -1] = 0
    out = p.infer(obs=_obs(), noise=torch.ones(H, AD), dof_mask=dof)
    assert eng.last["padding"].shape == (H, AD) and torch.allclose(out.extra["x_norm"][:, -1], torch.zeros(H))
    with pytest.raises(ValueError, match="dof_mask must contain only 0 or 1"):
        p.infer(obs=_obs(), dof_mask=torch.full((H, AD), 0.5))
    with pytest.raises(ValueError, match="noise shape"):
        p.infer(obs=_obs(), noise=torch.ones(H + 1, AD))
    with pytest.raises(ValueError, match="pass either obs"):
        p.infer(images=[1])
    with pytest.raises(UnsupportedModelError, match="rtc"):
        p.infer(obs=_obs(), use_rtc=True)
    n = eng.calls
    p.prepare_graphs(obs=_obs())                      # BUILD + REPLAY + determinism check + freeze
    assert eng.calls == n + 2 and p.graphs_ready and p.graph_profile["deterministic"] and p.graph_profile["num_steps"] == 10
    with pytest.raises(RuntimeError, match="already prepared"):
        p.prepare_graphs(obs=_obs())
    with pytest.raises(RPUBackendError, match="outside the prepared graph profile"):
        p.infer(obs=_obs(), num_steps=5)
    with pytest.raises(RPUBackendError, match="outside the prepared graph profile"):
        p.infer(obs=_obs(), dof_mask=dof)
    assert p.predict_action_chunk(obs=_obs()).shape == (H, AD)
    p.close()
    p.close()
    assert eng.closed
    with pytest.raises(RPUBackendError, match="closed"):
        p.infer(obs=_obs())
    with pytest.raises(RPUBackendError, match="non-finite"):
        WallOssPolicy._from_engine(_FakeEngine(nan=True)).infer(obs=_obs())


def test_active_slots_make_the_default_dof_mask():
    eng = _FakeEngine()
    p = WallOssPolicy._from_engine(eng, normalizer=_norm(), active_slots=[0, 2])
    out = p.infer(obs=_obs(), noise=torch.ones(eng.cfg.horizon, eng.cfg.action_dim))
    x = out.extra["x_norm"]
    assert torch.allclose(x[:, [0, 2]], torch.full((eng.cfg.horizon, 2), 0.5)) and torch.allclose(x[:, [1, 3, 4, 5]], torch.zeros(eng.cfg.horizon, 4))
    with pytest.raises(ValueError, match="exceeds action_dim"):
        WallOssPolicy._from_engine(eng, normalizer=_norm(), active_slots=[9]).infer(obs=_obs())


def test_prompt_state_string_and_normalizer():
    s = discretize_proprioception(np.array([-1.0, -0.999, 0.0, 0.999, 1.0]), 256)
    assert s == "0 0 128 255 255"
    assert discretize_proprioception(np.array([0.0]), 512) == "256"
    text = build_flow_prompt("open the drawer", ["face_view", "left_wrist_view"], "x2_berkeley_ur5", False, "1 2 3")
    assert text.startswith("<|im_start|>system\nYou are an embodied vision-language-action (VLA) model controlling the robot "
                           "with language instructions.\n Embodiment: ur5\n Camera Setup: front view, left wrist view,\n "
                           "Frequency: 32HZ\n Action Space: Abs EEF\n<|im_end|>\n<|im_start|>user\nObservation: front view: "
                           "<|vision_start|><|image_pad|><|vision_end|> left wrist view: <|vision_start|><|image_pad|><|vision_end|>\n"
                           "Instruction: open the drawer\nPredict the next action in robot action.\nProprioception: 1 2 3\n<|im_end|>\n")
    assert text.endswith("<|im_start|>assistant\n")
    assert "Rel EEF" in build_flow_prompt("x", ["face_view"], "d", True, "")
    short = build_flow_prompt("go", ["face_view", "top_view"], "d", False, "9", style="short")
    assert short == "<|im_start|>user\n" + "<|vision_start|><|image_pad|><|vision_end|>" * 2 + " go<|im_end|>\n<|im_start|>assistant\n"
    assert "Single Franka" in build_flow_prompt("x", ["face_view"], "d", False, "", style="multisuite")
    assert "Camera Setup: front view\nAction Space" in build_flow_prompt("x", ["face_view"], "d", False, "", style="generic")
    with pytest.raises(ValueError, match="unknown camera"):
        build_flow_prompt("x", ["nope"], "d", False, "")
    ex = expand_image_tokens("a<|image_pad|>b<|image_pad|>c", torch.tensor([[1, 4, 6], [1, 2, 2]]), 2)
    assert ex == "a" + "<|image_pad|>" * 6 + "b" + "<|image_pad|>" + "c"
    with pytest.raises(ValueError, match="image placeholders"):
        expand_image_tokens("a<|image_pad|>", torch.tensor([[1, 4, 6], [1, 2, 2]]), 2)
    n = _norm()
    assert n.state_string(torch.tensor([-1.0, 0.0, 5.0, 0.5]), torch.tensor([1, 1, 1, 0]), 256) == "0 128 255"
    assert torch.allclose(n.denormalize(torch.tensor([[-1.0, 1.0, 0.0, 0.0, 0.0, 0.0]])), torch.tensor([[-2.0, 2.0, 0, 0, 0, 0]]))
    assert torch.allclose(n.padding_action(3), torch.zeros(3, 6))
    from rhinoforge_b200.api import RPUConfigError
    with pytest.raises(RPUConfigError, match="no entry"):
        Normalizer({"min.a": torch.ones(1), "delta.a": torch.ones(1)}, {"min.a": torch.ones(1), "delta.a": torch.ones(1)}, "b")


def test_configuration_admission():
    flat = dict(vocab_size=200, hidden_size=2048, num_hidden_layers=36, num_attention_heads=16, num_key_value_heads=2,
                rope_theta=1e6, rope_scaling={"mrope_section": [16, 24, 24]}, action_hidden_size=1024,
                experts=[dict(hidden_size=2048, intermediate_size=11008), dict(hidden_size=1024, intermediate_size=2048)])
    t = text_config(flat)
    assert (t.hidden_size, t.intermediate_size, t.head_dim, t.mrope_section, t.mrope_interleaved, t.attention_bias, t.qk_norm) == \
        (2048, 11008, 128, (16, 24, 24), False, True, False)
    c = action_config(flat, action_dim=26)
    assert (c.hidden, c.inter, c.layers, c.heads, c.kv_heads, c.head_dim, c.action_dim) == (1024, 2048, 36, 16, 2, 128, 26)
    with pytest.raises(UnsupportedModelError, match="experts"):
        text_config({**flat, "experts": None})
    with pytest.raises(UnsupportedModelError, match="action_hidden_size"):
        action_config({**flat, "action_hidden_size": 512}, action_dim=26)
    with pytest.raises(UnsupportedModelError, match="mrope_section"):
        text_config({**flat, "rope_scaling": {}})
    # contiguous M-RoPE frequency ranges: 16 temporal, 24 row, 24 column pairs
    from rhinoforge_b200.models.decoder import mrope_axis_of_freq
    ax = mrope_axis_of_freq(t)
    assert ax.tolist() == [0] * 16 + [1] * 24 + [2] * 24


def test_schedule_pieces_match_their_definitions():
    cfg = tiny_wall_oss_config()
    sd = random_wall_oss_expert(cfg, seed=1, dtype=torch.float32)
    assert torch.allclose(flow_times(4), torch.tensor([0.0, 0.25, 0.5, 0.75, 1.0]))
    e = sinusoidal_pos_emb(torch.tensor([0.3]), 64)
    f = torch.exp(torch.arange(32, dtype=torch.float32) * -(np.log(10000.0) / 31))
    assert torch.allclose(e[0, :32], torch.sin(0.3 * f)) and torch.allclose(e[0, 32:], torch.cos(0.3 * f))
    w, sb = folded_preprocessor(sd, cfg, 4)
    x = torch.randn(cfg.horizon, 2 * cfg.action_dim)
    for k in range(4):
        te = sinusoidal_pos_emb(flow_times(4)[k:k + 1], cfg.hidden).expand(cfg.horizon, -1)
        want = F.linear(torch.cat((F.linear(x, sd[PRE_P + "w1.weight"]), te), -1), sd[PRE_P + "w2.weight"])
        assert float((x @ w.t() + sb[k] - want).abs().max()) < 1e-5
    m = action_mask(5, 3, 10, causal=True)
    assert m.int().tolist() == [[1] * 5 + [1, 0, 0, 0, 0], [1] * 5 + [1, 1, 0, 0, 0], [1] * 5 + [1, 1, 1, 0, 0]]
    assert action_mask(5, 3, 10, causal=False).int().tolist() == [[1] * 8 + [0, 0]] * 3
    noise, dof = torch.randn(3, 4), torch.ones(3, 4)
    assert masked_dof_inputs(noise, dof, None) == (None, None)
    dof[:, 3] = 0
    with pytest.raises(ValueError, match="padding_action is required"):
        masked_dof_inputs(noise, dof, None)
    pad = torch.full((3, 4), 0.25)
    mk, ovr = masked_dof_inputs(noise, dof, pad)
    assert torch.equal(mk, dof) and torch.allclose(ovr[:, 3], 0.25 - noise[:, 3]) and float(ovr[:, :3].abs().max()) == 0.0
    # Euler over the unit interval with the blend lands inactive dimensions exactly on the padding action
    x = noise.clone()
    for _ in range(4):
        x = x + 0.25 * (torch.randn(3, 4) * mk + ovr)
    assert torch.allclose(x[:, 3], pad[:, 3], atol=1e-6)


def test_checkpoint_name_translation():
    cfg = tiny_wall_oss_config()
    flat = dict(vocab_size=50, hidden_size=96, num_hidden_layers=cfg.layers, num_attention_heads=cfg.heads,
                num_key_value_heads=cfg.kv_heads, head_dim=cfg.head_dim, rope_scaling={"mrope_section": [8, 12, 12]},
                experts=[dict(hidden_size=96, intermediate_size=160), dict(hidden_size=cfg.hidden, intermediate_size=cfg.inter)])
    t = text_config(flat)
    g = torch.Generator().manual_seed(0)
    sd = {n: torch.randn(s, generator=g) for n, s, _ in wall_oss_expert_shapes(cfg, 0, hidden=96, inter=160)}
    sd["model.embed_tokens.weight"] = torch.randn(50, 96, generator=g)
    get = expert0_getter(lambda n: sd[n], t, set(sd))
    hd, nq, nkv = cfg.head_dim, cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    qkv = sd["model.layers.1.self_attn.qkv_proj_experts.0.weight"]
    assert torch.equal(get("model.layers.1.self_attn.q_proj.weight"), qkv[:nq])
    assert torch.equal(get("model.layers.1.self_attn.k_proj.weight"), qkv[nq:nq + nkv])
    assert torch.equal(get("model.layers.1.self_attn.v_proj.bias"), sd["model.layers.1.self_attn.qkv_proj_experts.0.bias"][nq + nkv:])
    gu = sd["model.layers.0.moe.experts.0.gate_up_proj.weight"]
    assert torch.equal(get("model.layers.0.mlp.gate_proj.weight"), gu[:160]) and torch.equal(get("model.layers.0.mlp.up_proj.weight"), gu[160:])
    assert torch.equal(get("model.norm.weight"), sd["model.norms.0.weight"])
    assert torch.equal(get("lm_head.weight"), sd["model.embed_tokens.weight"])           # no separate head: tied
    with pytest.raises(KeyError):
        get("model.layers.0.self_attn.q_norm.weight")
    # vision: fused gate/up halves, each zero-padded past the logical width
    vs = {"visual.blocks.0.mlp.gate_up_proj.weight": torch.cat((torch.ones(5, 3), torch.zeros(1, 3), 2 * torch.ones(5, 3), torch.zeros(1, 3))),
          "visual.blocks.0.mlp.down_proj.weight": torch.ones(3, 6), "visual.merger.ln_q.weight": torch.ones(3)}
    vn = VisionNames(lambda n: vs[n], 5)
    assert torch.equal(vn["blocks.0.mlp.gate_proj.weight"], torch.ones(5, 3)) and torch.equal(vn["blocks.0.mlp.up_proj.weight"], 2 * torch.ones(5, 3))
    assert vn["blocks.0.mlp.down_proj.weight"].shape == (3, 5) and torch.equal(vn["merger.ln_q.weight"], torch.ones(3))
