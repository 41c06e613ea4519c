"""Host-only checks of the weight layout rule, the chunk envelope, rotary table builders, the attribute guard,
the tile-major packer and the Pi0.5 facade's input plumbing."""
import pytest
import torch


def test_linear_partition_rule_and_shards():
    from rhinoforge_b200.runtime import weights as W
    assert W.get_linear_partition(4096, 12288, 2, 8, "model.layers.0.mlp.gate_proj") == W.PARTITION_COL
    assert W.get_linear_partition(12288, 4096, 2, 8, "model.layers.0.mlp.down_proj") == W.PARTITION_ROW
    assert W.get_linear_partition(4096, 4096, 2, 8, "model.layers.3.self_attn.o_proj") == W.PARTITION_ROW
    assert W.get_linear_partition(100, 30, 2, 8, "head") == W.PARTITION_HOST
    w = torch.arange(8 * 16, dtype=torch.float32).view(8, 16)
    assert torch.equal(W.shard_linear(w, W.PARTITION_COL, 1, 4), w[2:4])
    assert torch.equal(W.shard_linear(w, W.PARTITION_ROW, 3, 4), w[:, 12:16])
    plan = W.partition_plan([("a.q_proj", (64, 32)), ("a.o_proj", (32, 64))], 8)
    assert plan == {"a.q_proj": 1, "a.o_proj": 0}


def test_pack_weight_layout_matches_the_swizzle_rule():
    from rhinoforge_b200.ops.kernels import pack_weight
    w = torch.arange(130 * 70, dtype=torch.float16).view(130, 70)
    p = pack_weight(w).view(2, 2, 128, 64)                       # [row tile, k block, row, col]
    for (r, c) in ((5, 9), (129, 67), (0, 0), (127, 63)):
        rt, rr, kb, cc = r // 128, r % 128, c // 64, c % 64
        chunk, within = cc // 8, cc % 8
        assert p[rt, kb, rr, ((chunk ^ (rr % 8)) * 8) + within] == w[r, c]
    assert float(p[1, 1, 5].abs().sum()) == 0.0                  # padding rows are zero
    q = torch.randint(-127, 128, (256, 128), dtype=torch.int8)
    pq = pack_weight(q, 2).view(2, 2, 128, 64)                    # int8: plain row-major blocks, two sections
    assert torch.equal(pq[1, 1], q[128:256, 64:128])


def test_chunk_envelope():
    from rhinoforge_b200.runtime.chunk_envelope import ChunkEnvelope
    e = ChunkEnvelope(4096, 512)
    assert (e.pages, e.chunks_for(1000)) == (256, 2)
    assert e.admits(4000, 96) and not e.admits(4000, 100)
    with pytest.raises(ValueError):
        ChunkEnvelope(4096, 100)
    with pytest.raises(ValueError):
        e.check(4096, 1)


def test_rope_builders_agree_with_each_other():
    from rhinoforge_b200.runtime import rope_partial as R
    axis = R.mrope_axis_of_freq(64, (11, 11, 10))
    assert axis.tolist()[:7] == [0, 1, 2, 0, 1, 2, 0] and int((axis == 0).sum()) == 11
    assert int((axis == 1).sum()) == 11 and int((axis == 2).sum()) == 10
    cos, sin = R.rope_tables(64, 50, 1e4)
    pos3 = torch.stack((torch.arange(20), torch.arange(20) + 3, torch.arange(20) + 7))
    bc, bs = R.baked_interleaved_tables(pos3, 64, (11, 11, 10), 1e4)
    f = torch.arange(32)
    want = cos[pos3[axis.long(), :].t(), f]
    assert torch.allclose(bc, want, atol=1e-6)
    assert R.partial_rotary_dim(256, 0.25) == 64
    with pytest.raises(ValueError):
        R.mrope_axis_of_freq(64, (10, 10, 10))


def test_attribute_guard():
    from rhinoforge_b200.runtime import hw_attrs
    from rhinoforge_b200.runtime.errors import RPUConfigError

    @hw_attrs.guard
    class Handle:
        pass
    h = Handle()
    h._rpu_execution = {"prefill": {"chunk_size": 512}}
    h._rpu_last_execution_plan = {"stage": "prefill"}
    h._rpu_freeze()
    h._rpu_last_execution_plan = {"stage": "decode"}             # public: always writable
    h._rpu_execution = {"prefill": {"chunk_size": 512}}          # same value: allowed
    with pytest.raises(RPUConfigError):
        h._rpu_execution = {"prefill": {"chunk_size": 256}}
    with pytest.raises(RPUConfigError):
        h._rpu_typo = 1
    with pytest.raises(RPUConfigError):
        h._rpu_is_ready = False
    assert hw_attrs.classify("other") == "foreign"


def test_pi05_image_preprocessing_and_checkpoint_names():
    from rhinoforge_b200.adapters.pi05 import canonical_name, config_from_policy_config
    from rhinoforge_b200.api.policy import resize_with_pad
    img = torch.rand(2, 3, 100, 200)
    out = resize_with_pad(img, 224)
    assert out.shape == (2, 3, 224, 224)
    assert float(out[:, :, :50].max()) == -1.0 and float(out[:, :, -50:].max()) == -1.0       # padded bands are black
    assert -1.0 <= float(out.min()) and float(out.max()) <= 1.0
    same = resize_with_pad(torch.rand(1, 3, 224, 224), 224)
    assert same.shape == (1, 3, 224, 224)
    assert canonical_name("model.paligemma_with_expert.gemma_expert.model.norm.dense.weight") == \
        "paligemma_with_expert.gemma_expert.model.norm.dense.weight"
    cfg, meta = config_from_policy_config({"chunk_size": 50, "max_action_dim": 32, "n_action_steps": 25,
                                           "input_features": {"observation.images.a": {}, "observation.images.b": {},
                                                              "observation.images.c": {}, "observation.state": {}},
                                           "output_features": {"action": {"shape": [7]}}})
    assert (cfg.num_views, cfg.horizon, cfg.action_dim) == (3, 50, 32)
    assert meta == {"camera_keys": ["observation.images.a", "observation.images.b", "observation.images.c"],
                    "n_action_steps": 25, "action_dim": 7}


def test_pi05_oracle_runs_on_cpu_and_ignores_masked_inputs():
    """The padded/masked reference is insensitive to what sits in masked cameras and padded tokens."""
    from rhinoforge_b200.models.pi05 import TorchPi05, random_pi05_state_dict, tiny_pi05_config
    cfg = tiny_pi05_config()
    sd = random_pi05_state_dict(cfg, dtype=torch.float32, std=0.08, seed=1)
    m = TorchPi05(cfg, sd)
    g = torch.Generator().manual_seed(0)
    img = torch.randn(1, cfg.num_views, 3, 56, 56, generator=g)
    imask = torch.tensor([[True, False]])
    tok = torch.randint(0, cfg.vocab_size, (1, 10), generator=g)
    tmask = torch.arange(10)[None] < 7
    noise = torch.randn(1, cfg.horizon, cfg.action_dim, generator=g)
    a = m.sample_actions(img, imask, tok, tmask, noise, 3)
    img2, tok2 = img.clone(), tok.clone()
    img2[:, 1] = 5.0
    tok2[:, 7:] = 3
    b = m.sample_actions(img2, imask, tok2, tmask, noise, 3)
    assert torch.allclose(a, b, atol=1e-5)


def test_action_denormalizer_and_runtime_env():
    import numpy as np
    from rhinoforge_b200.api._runtime_env import normalize_runtime_env
    from rhinoforge_b200.api.action_denorm import ActionDenormalizer, ActionGroup
    groups = [ActionGroup("arm", 3, "meanstd"), ActionGroup("grip", 1, "minmax"),
              ActionGroup("base", 2, "bounds_99_woclip", subtract_state=True, state_key="observation.state.base")]
    stats = {"arm": {"mean": np.array([1.0, 2.0, 3.0]), "std": np.array([0.5, 0.5, 2.0])},
             "grip": {"min": np.array([0.0]), "max": np.array([0.08])},
             "base": {"q01": np.array([-1.0, -2.0]), "q99": np.array([1.0, 2.0])}}
    d = ActionDenormalizer(groups, stats)
    a = torch.tensor([[1.0, -1.0, 0.0, 3.0, 0.5, -2.0, 9.0]])            # trailing padding column is ignored
    out = d(a, {"observation.state.base": np.array([10.0, 20.0])})
    assert out.shape == (1, 6)
    assert np.allclose(out[0, :3], [1.5, 1.5, 3.0], atol=1e-5)
    assert np.isclose(out[0, 3], (3.0 + 1) / 2 * 0.08, atol=1e-5)        # the inverse never clips: 3.0 maps past max
    assert np.allclose(out[0, 4:], [10.5, 16.0], atol=1e-4)              # no clip, delta added
    with pytest.raises(ValueError):
        ActionDenormalizer([ActionGroup("x", 2, "sincos")], {})
    with pytest.raises(KeyError):
        ActionDenormalizer([ActionGroup("x", 2, "meanstd")], {"x": {"mean": np.zeros(2)}})
    env = normalize_runtime_env({"RPU_WARMUP": 1}, owner="policy", allowed={"RPU_WARMUP"})
    assert env == {"RPU_WARMUP": "1"}
    with pytest.raises(ValueError, match="before importing"):
        normalize_runtime_env({"RPU_LOG_LEVEL": 3}, owner="policy", allowed={"RPU_WARMUP"})
    with pytest.raises(ValueError, match="unsupported"):
        normalize_runtime_env({"PATH": "x"}, owner="policy", allowed={"RPU_WARMUP"})


def test_rotation_6d_decode_roundtrip():
    import numpy as np
    from rhinoforge_b200.api import hy_action_decode as H
    rng = np.random.default_rng(0)
    q = rng.normal(size=(5, 4))
    R = H.quat_xyzw_to_matrix(q)
    assert np.allclose(R @ np.swapaxes(R, -1, -2), np.eye(3), atol=1e-9)
    d6 = np.concatenate((R[..., 0, :], R[..., 1, :]), -1)             # the encoding is the first two ROWS
    assert np.allclose(H.rotation_6d_to_matrix(d6), R, atol=1e-9) and np.allclose(H.matrix_to_rotation_6d(R), d6)
    q2 = H.matrix_to_quat_xyzw(R)
    assert np.allclose(H.quat_xyzw_to_matrix(q2), R, atol=1e-9)
    start = np.array([0.1, 0.2, 0.3, 0.0, 0.0, 0.0, 1.0])
    rel = np.zeros((2, 10)); rel[:, 3] = 1.0; rel[:, 7] = 1.0; rel[1, :3] = [1, 0, 0]; rel[:, 9] = 0.5
    poses = H.relative_to_absolute_poses(rel, start)
    assert np.allclose(poses[0], [0.1, 0.2, 0.3, 0, 0, 0, 1, 0.5]) and np.allclose(poses[1, :3], [1.1, 0.2, 0.3])
    assert H.relative_to_dual_arm_poses(np.concatenate((rel, rel), 1), np.concatenate((start, start))).shape == (2, 16)
    sixteen = np.concatenate((start, [0.0], start + [1.0, 1.0, 1.0, 0, 0, 0, 0], [0.0]))
    dual = H.relative_to_dual_arm_poses(np.concatenate((rel, rel), 1), sixteen)
    assert np.allclose(dual[1, :3], [1.1, 0.2, 0.3]) and np.allclose(dual[1, 8:11], [2.1, 1.2, 1.3])
    with pytest.raises(ValueError, match="16 wide"):
        H.relative_to_dual_arm_poses(np.concatenate((rel, rel), 1), np.zeros(15))


def test_hy_vla_action_decoder_matches_a_scipy_statement_of_the_contract():
    import numpy as np
    from scipy.spatial.transform import Rotation as Rot
    from rhinoforge_b200.api.hy_action_decode import HyVlaActionDecoder, convert_frame, quat_wxyz_to_xyzw, quat_xyzw_to_wxyz
    rng = np.random.default_rng(3)
    H = 6
    stats = {"action_mean": rng.normal(size=(H, 20)) * 0.01, "action_std": rng.uniform(0.5, 1.5, size=(H, 20)),
             "qpos_mean": rng.normal(size=20) * 0.1, "qpos_std": rng.uniform(0.5, 1.5, size=20)}
    W = np.array([[0, 1, 0], [-1, 0, 0], [0, 0, 1.0]])
    P = np.array([[0, 0, 1], [1, 0, 0], [0, 1, 0.0]])

    def unit(q):
        return q / np.linalg.norm(q)
    start_wxyz = np.concatenate(([0.3, -0.1, 0.5], unit(rng.normal(size=4)), [0.7],
                                 [-0.2, 0.4, 0.6], unit(rng.normal(size=4)), [0.2]))
    act = rng.normal(size=(1, H, 32)) * 0.3
    for arm in (3, 13):                                               # keep the two encoded rows far from parallel
        act[0, :, arm:arm + 6] += np.array([3.0, 0, 0, 0, 3.0, 0])

    def by_scipy(umi: bool, grip: bool, drop: bool):
        rel = act[0, :, :20] * stats["action_std"] + stats["action_mean"]
        out = np.zeros((H, 16))
        for a_off, p_off in ((0, 0), (10, 8)):
            t0 = start_wxyz[p_off:p_off + 3]
            R0 = Rot.from_quat(start_wxyz[p_off + 3:p_off + 7][[1, 2, 3, 0]]).as_matrix()
            g0 = start_wxyz[p_off + 7]
            if umi:
                t0, R0 = W @ t0, W @ R0 @ P
            for h in range(H):
                r1 = rel[h, a_off + 3:a_off + 6]; r2 = rel[h, a_off + 6:a_off + 9]
                b1 = r1 / np.linalg.norm(r1); b2 = r2 - (b1 @ r2) * b1; b2 /= np.linalg.norm(b2)
                dR = np.stack((b1, b2, np.cross(b1, b2)))              # rows
                R, t, g = R0 @ dR, t0 + R0 @ rel[h, a_off:a_off + 3], rel[h, a_off + 9]
                if umi:
                    t, R = W.T @ t, W.T @ R @ P.T
                    if grip:
                        g = 1.0 - g / 90.0
                out[h, p_off:p_off + 3] = t
                out[h, p_off + 3:p_off + 7] = Rot.from_matrix(R).as_quat()[[3, 0, 1, 2]]
                out[h, p_off + 7] = g
        return out[1:] if drop else out

    def same_pose(a, b):
        a, b = a.copy(), b.copy()
        for s in (3, 11):                                             # q and -q are the same rotation
            flip = np.sign((a[:, s:s + 4] * b[:, s:s + 4]).sum(-1, keepdims=True))
            b[:, s:s + 4] *= flip
        return np.allclose(a, b, atol=1e-9)

    for umi, grip, drop in ((True, False, True), (False, False, False), (True, True, True)):
        dec = HyVlaActionDecoder.from_norm_stats_mapping(stats, umi_coord_frame=umi, umi_gripper_space=grip, drop_first=drop)
        got = dec.decode(act, start_wxyz)
        assert got.shape == ((H - 1) if drop else H, 16) and same_pose(got, by_scipy(umi, grip, drop)), (umi, grip, drop)
    dec = HyVlaActionDecoder.from_norm_stats_mapping(stats)
    assert dec.horizon == H and dec.decode(act[0, :3, :20], start_wxyz).shape == (2, 16)

    # state encoding: frame change, rows of the rotation, then (x - mean) / (std + 1e-8)
    st = dec.encode_state(start_wxyz)
    assert st.shape == (1, 20)
    raw = st[0] * (stats["qpos_std"] + 1e-8) + stats["qpos_mean"]
    Rl = W @ Rot.from_quat(start_wxyz[3:7][[1, 2, 3, 0]]).as_matrix() @ P
    assert np.allclose(raw[:3], W @ start_wxyz[:3]) and np.allclose(raw[3:9], np.concatenate((Rl[0], Rl[1])), atol=1e-9)
    assert np.isclose(raw[9], 0.7) and np.isclose(raw[19], 0.2)

    # frame change and quaternion order are invertible
    p = quat_wxyz_to_xyzw(start_wxyz)[None]
    back = convert_frame(convert_frame(p, to_umi=True, convert_gripper=True), to_umi=False, convert_gripper=True)
    assert same_pose(back, p) and np.allclose(quat_xyzw_to_wxyz(p)[0], start_wxyz)
    assert np.isclose(convert_frame(p, to_umi=True, convert_gripper=True)[0, 7], (1 - 0.7) * 90)

    for bad, exc, msg in ((dict(action_mean=np.zeros((4, 19)), action_std=np.zeros((4, 19))), ValueError, r"\[H, 20\]"),
                          (dict(action_mean=np.zeros((4, 20)), action_std=np.zeros((5, 20))), ValueError, "differ in shape"),
                          (dict(action_mean=np.zeros((4, 20))), KeyError, "action_std"),
                          ({**stats, "action_mean_abs": 1, "action_std_abs": 1}, NotImplementedError, "absolute and relative")):
        with pytest.raises(exc, match=msg):
            HyVlaActionDecoder.from_norm_stats_mapping(bad)
    with pytest.raises(TypeError):
        HyVlaActionDecoder.from_norm_stats_mapping([1, 2])
    with pytest.raises(ValueError, match="requires umi_coord_frame"):
        HyVlaActionDecoder(stats["action_mean"], stats["action_std"], umi_coord_frame=False, umi_gripper_space=True)
    for bad_act, msg in ((np.zeros((2, H, 20)), "batch 1"), (np.zeros((H + 1, 20)), "exceed"), (np.zeros((H, 19)), "at least 20")):
        with pytest.raises(ValueError, match=msg):
            dec.decode(bad_act, start_wxyz)
    with pytest.raises(ValueError, match="16 entries"):
        dec.decode(act, start_wxyz[:14])
    with pytest.raises(ValueError, match="cannot be encoded"):
        HyVlaActionDecoder(stats["action_mean"], stats["action_std"]).encode_state(start_wxyz)


def test_qwen25vl_window_partition_matches_hf_index():
    """The window-major unit order and window sizes equal the Hugging Face module's ``get_window_index`` (ragged
    edge windows, several frames, several images)."""
    import torch
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig as HFConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel as HFModel
    from rhinoforge_b200.models.qwen25_vl_vision import window_partition

    hc = HFConfig(depth=1, hidden_size=32, num_heads=2, intermediate_size=32, patch_size=14, temporal_patch_size=2,
                  spatial_merge_size=2, out_hidden_size=16, window_size=112, fullatt_block_indexes=[0])
    ref = HFModel(hc)
    for grid in ([[1, 6, 10]], [[2, 4, 4], [1, 18, 22]], [[3, 10, 26], [1, 2, 2]]):
        idx, cu = ref.get_window_index(torch.tensor(grid))
        cu = torch.unique_consecutive(torch.tensor(cu))
        order, lens = window_partition([tuple(g) for g in grid], 2, 112 // 2 // 14)
        assert order == [int(i) for i in idx]
        assert [4 * n for n in lens] == (cu[1:] - cu[:-1]).tolist()


def test_signature_planner_layers_and_miss_attribution():
    import torch
    from rhinoforge_b200.graph.admission import SignaturePlanner

    P = SignaturePlanner()
    x = torch.zeros(2, 5, 8)

    def f(a):
        return a

    base = P.layers_for_call("op", (x, 3), {"flag": True}, branch=f)
    assert P.layers_for_call("op", (torch.zeros(2, 5, 8), 3), {"flag": True}, branch=f) == base
    cases = {
        "gm_id": P.layers_for_call("other", (x, 3), {"flag": True}, branch=f),
        "tensor_struct": P.layers_for_call("op", ((x, x), 3), {"flag": True}, branch=f),
        "shape_bucket": P.layers_for_call("op", (torch.zeros(2, 6, 8), 3), {"flag": True}, branch=f),
        "dtype_layout": P.layers_for_call("op", (x.half(), 3), {"flag": True}, branch=f),
        "scalar_flags": P.layers_for_call("op", (x, 4), {"flag": True}, branch=f),
        "branch_key": P.layers_for_call("op", (x, 3), {"flag": True}, branch=len),
        "segment_key": P.layers_for_call("op", (x, 3), {"flag": True}, branch=f, segment=2),
    }
    for reason, layers in cases.items():
        assert P.attribute_miss_reason(layers, [base]) == reason, reason
    assert P.attribute_miss_reason(base, []) == "no_entry"
    # the closest entry decides: one entry differs in the op, another only in a scalar
    assert P.attribute_miss_reason(cases["scalar_flags"], [cases["gm_id"], base]) == "scalar_flags"
    assert P.infer_workload_kind((torch.zeros(4, 1, 8),)) == "decode"
    assert P.infer_workload_kind((torch.zeros(4, 7, 8),)) == "prefill"
    assert P.infer_workload_kind((3, "x")) == "generic"
    assert P.stable_branch_key(f) == P.stable_branch_key(f) != P.stable_branch_key(len)
    assert P.stable_branch_key(None) == 0


def test_entry_registry_lru_and_plans_without_a_device():
    import torch
    from rhinoforge_b200.graph.admission import EntryRegistry, GraphPlan

    class FakeCache:          # the registry only needs this much of a GraphCache
        def __init__(self):
            self.evicted, self.frozen = [], False
        def is_frozen(self): return self.frozen
        def evict(self, sig): self.evicted.append(sig)
        def capture(self, sig): return ("scope", sig)
        def explain_miss(self, sig): return "miss"
        def size(self): return 0
        def clear(self): pass

    fc = FakeCache()
    reg = EntryRegistry(fc, max_entries=2)
    # without the native backend every signature hashes alike, so give each plan its own key object
    class Sig:
        def __init__(self, k): self.k, self._impl = k, (k,)
        def __hash__(self): return hash(self.k)
        def __eq__(self, o): return self.k == o.k
    L = reg.planner.layers_for_call("op", (torch.zeros(1, 1),))
    plans = [GraphPlan(Sig(i), L) for i in range(3)]
    for p in plans[:2]:
        assert reg.admit_for_call(p)[0] == "scope" and p.admission == "record"
    assert reg.admit_for_call(plans[0]) and plans[0].admission == "replay"
    reg.admit_for_call(plans[2])                       # evicts plans[1] (least recently used)
    assert fc.evicted == [plans[1].signature] and plans[2].lifecycle == "evict"
    st = reg.stats()
    assert (st["hits"], st["misses"], st["evictions"], st["entries"]) == (1, 3, 1, 2)
    fc.frozen = True
    import pytest
    with pytest.raises(RuntimeError, match="frozen"):
        reg.admit_for_call(GraphPlan(Sig(9), L))
    assert "plan[" in plans[2].to_log_str()


def test_manual_capture_passes_through_without_a_device_and_refuses_drift():
    import pytest
    import torch
    from rhinoforge_b200.graph import capture

    calls = []

    def fn(a, b, *, k=2):
        calls.append(1)
        return a * k + b

    a, b = torch.ones(3), torch.arange(3.0)
    g = capture(fn, a, b, k=2)
    if not torch.cuda.is_available():
        assert not g.replayable and g.non_replayable_reason
        assert torch.equal(g.replay(a, b, k=2), a * 2 + b)
        assert g.stats()["passthrough_calls"] == 1 and len(calls) == 2
    with pytest.raises(RuntimeError, match="shape_bucket"):
        g.replay(torch.ones(4), torch.ones(4), k=2)
    with pytest.raises(RuntimeError, match="scalar_flags"):
        g.replay(a, b, k=3)
    with pytest.raises(NotImplementedError):
        capture(fn, a, b, dynamic_inputs=("a",))
    g.invalidate()
    with pytest.raises(RuntimeError, match="invalidated"):
        g.replay(a, b, k=2)


def test_bounded_prefill_planner_orders_launches_then_padding_then_deficit():
    import pytest
    from rhinoforge_b200.runtime.decoder import (chunk_policy_key, default_chunk_resolver, plan_bounded_prefill_execution,
                                                 prefill_position_key)
    res = default_chunk_resolver(256)
    assert plan_bounded_prefill_execution(100, 4096, 64, res) == (100, 112)            # one launch, no padding needed
    assert plan_bounded_prefill_execution(300, 4096, 64, res) == (300, 256)            # two launches either way: keep raw rows
    assert plan_bounded_prefill_execution(100, 4096, 64, res, alignment=64) == (128, 128)
    assert plan_bounded_prefill_execution(100, 4096, 0, res, padding_rows=12) == (112, 112)
    # a resolver with a coarse grid: padding is taken only because it saves a launch
    grid = lambda n: 128 if n % 128 == 0 else 64
    assert plan_bounded_prefill_execution(120, 4096, 16, grid) == (128, 128)
    assert plan_bounded_prefill_execution(120, 4096, 4, grid) == (120, 64)
    # exact chunk requests, the padding-only launch rule, limits and bad arguments
    assert plan_bounded_prefill_execution(120, 4096, 16, grid, exact_chunk_size=128) == (128, 128)
    with pytest.raises(ValueError, match="not the requested"):
        plan_bounded_prefill_execution(100, 4096, 0, res, exact_chunk_size=256)
    with pytest.raises(ValueError, match="padding only"):
        plan_bounded_prefill_execution(60, 4096, 0, lambda n: 64, padding_rows=68)
    with pytest.raises(ValueError, match="physical limit"):
        plan_bounded_prefill_execution(100, 150, 0, res, position=100)
    with pytest.raises(ValueError, match="multiple of 16"):
        plan_bounded_prefill_execution(100, 4096, 0, res, exact_chunk_size=100)
    with pytest.raises(ValueError, match="alignment"):
        plan_bounded_prefill_execution(100, 4096, 0, res, alignment=64, padding_rows=1)
    score = lambda n, c, launches, pad, deficit: (pad, launches)                        # caller prefers no padding at all
    assert plan_bounded_prefill_execution(120, 4096, 16, grid, candidate_score=score) == (120, 64)
    assert chunk_policy_key("auto") == 0 and chunk_policy_key(None) == 0 and chunk_policy_key(512) == 512
    assert prefill_position_key(1, 900) == 0 and prefill_position_key(32, 0) == 0 and prefill_position_key(32, 64) == 64


def test_every_builtin_adapter_in_the_manifest_imports():
    """The manifest is data only; every row must resolve to a class (a row for a family that is not built would make
    ``get_adapter`` fail with an import error instead of a model error)."""
    from rhinoforge_b200.adapters._manifest import BUILTIN_ADAPTERS
    from rhinoforge_b200.runtime.registry import get_adapter
    for arch, module, cls in BUILTIN_ADAPTERS:
        got = get_adapter(arch)
        assert got.__name__ == cls and got.__module__.startswith(module)


def test_vision_tower_adapters_preflight_from_the_config_alone():
    import pytest
    from rhinoforge_b200.adapters.hyvit2 import HYViT2Adapter
    from rhinoforge_b200.adapters.qwen25_vl_vision import Qwen25VLVisionAdapter
    from rhinoforge_b200.runtime.errors import UnsupportedModelError
    ok = dict(depth=32, hidden_size=1280, num_heads=16, intermediate_size=3420, patch_size=14, spatial_merge_size=2,
              window_size=112, fullatt_block_indexes=[7, 15, 23, 31], hidden_act="silu")
    Qwen25VLVisionAdapter.preflight(ok)
    for bad in (dict(ok, hidden_act="gelu"), dict(ok, window_size=100), dict(ok, fullatt_block_indexes=[40]),
                dict(ok, hidden_size=8192, num_heads=16)):
        with pytest.raises(UnsupportedModelError):
            Qwen25VLVisionAdapter.preflight(bad)
    HYViT2Adapter.preflight(dict(hidden_size=1152, num_attention_heads=16, image_size=224, patch_size=14))
    with pytest.raises(UnsupportedModelError):
        HYViT2Adapter.preflight(dict(hidden_size=1152, num_attention_heads=16, image_size=230, patch_size=14))


def test_evaluation_gates_and_model_switches_read_their_environment(monkeypatch):
    """Fail-closed gates admit only the exact literal 1; per-model switches use the strict boolean parser."""
    import pytest
    from types import SimpleNamespace as NS
    from rhinoforge_b200.adapters.qwen3_vl import Qwen3VLAdapter
    from rhinoforge_b200.runtime.errors import UnsupportedModelError
    text = dict(model_type="qwen3_vl_text", vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                num_attention_heads=64, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                rope_parameters={"rope_theta": 5e6, "mrope_section": [24, 20, 20]}, max_position_embeddings=262144)
    vision = dict(hidden_size=1024, intermediate_size=4096, depth=24, num_heads=16, patch_size=16, temporal_patch_size=2,
                  spatial_merge_size=2, out_hidden_size=5120, num_position_embeddings=2304,
                  deepstack_visual_indexes=[5, 11, 17], hidden_act="gelu_pytorch_tanh")
    cfg = NS(text_config=NS(**text), vision_config=NS(**vision), architectures=["Qwen3VLForConditionalGeneration"])
    monkeypatch.delenv("QWEN3_VL_32B_ALLOW_GRAPH_BLOCKED", raising=False)
    with pytest.raises(UnsupportedModelError, match="evaluation-gated"):
        Qwen3VLAdapter.preflight(cfg)
    monkeypatch.setenv("QWEN3_VL_32B_ALLOW_GRAPH_BLOCKED", "true")          # not the exact literal
    with pytest.raises(UnsupportedModelError, match="evaluation-gated"):
        Qwen3VLAdapter.preflight(cfg)
    monkeypatch.setenv("QWEN3_VL_32B_ALLOW_GRAPH_BLOCKED", "1")
    Qwen3VLAdapter.preflight(cfg)
    from rhinoforge_b200.runtime.control import rpu_env_bool, warmup_iters
    monkeypatch.setenv("RPU_PI05_DENOISE_UNROLL", "maybe")
    with pytest.raises(ValueError):
        rpu_env_bool("RPU_PI05_DENOISE_UNROLL", True)
    monkeypatch.setenv("RPU_WARMUP", "2")
    assert warmup_iters() == 2


def test_pi05_loader_ignores_a_stale_remapped_cache_file(tmp_path):
    import json
    import torch
    from safetensors.torch import save_file
    from rhinoforge_b200.adapters.pi05 import load_checkpoint
    (tmp_path / "config.json").write_text(json.dumps({"type": "pi05"}))
    save_file({"model.action_in_proj.weight": torch.ones(2, 2)}, str(tmp_path / "model.safetensors"))
    save_file({"action_in_proj.weight": torch.zeros(2, 2)}, str(tmp_path / "model_remapped.safetensors"))   # stale copy
    _, sd, _ = load_checkpoint(str(tmp_path))
    assert torch.equal(sd["action_in_proj.weight"], torch.ones(2, 2))


def test_chunked_gated_delta_rule_equals_the_recurrence():
    """The block-parallel form (triangular solve per chunk) reproduces the token-by-token recurrence: ragged last chunk,
    carried-in state, strong and weak decay, and agreement with the Hugging Face recurrent reference."""
    import torch
    from rhinoforge_b200.models.gdn_chunked import chunked_gated_delta_rule, recurrent_gated_delta_rule
    torch.manual_seed(0)
    T, H, Dk, Dv = 150, 3, 16, 24
    q = torch.nn.functional.normalize(torch.randn(T, H, Dk), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(T, H, Dk), dim=-1)
    v = torch.randn(T, H, Dv)
    g = -torch.rand(T, H) * 0.5
    g[40:60] *= 8.0                                         # a stretch of strong forgetting
    beta = torch.rand(T, H)
    s0 = torch.randn(H, Dk, Dv) * 0.3
    o_ref, s_ref = recurrent_gated_delta_rule(q, k, v, g, beta, state=s0)
    for chunk in (64, 32, 7):
        o, s = chunked_gated_delta_rule(q, k, v, g, beta, state=s0, chunk=chunk)
        assert torch.allclose(o, o_ref, atol=2e-4, rtol=2e-4), chunk
        assert torch.allclose(s, s_ref, atol=2e-4, rtol=2e-4), chunk
    try:
        from transformers.models.qwen3_next.modeling_qwen3_next import torch_recurrent_gated_delta_rule as hf
    except Exception:  # noqa: BLE001
        return
    o_hf, s_hf = hf(q[None], k[None], v[None], g[None], beta[None], initial_state=s0[None], output_final_state=True,
                    use_qk_l2norm_in_kernel=False)
    assert torch.allclose(o_hf[0].float(), o_ref, atol=2e-4, rtol=2e-4)
    assert torch.allclose(s_hf[0].float(), s_ref, atol=2e-4, rtol=2e-4)


def test_widened_int8_image_equals_the_packed_16bit_image_index_for_index():
    """The device pass that widens a tile-major int8 weight image writes piece ``c`` (8 values) of row ``r`` of a block
    to byte ``r*128 + ((c ^ (r & 7)) << 4)`` of the 16 KB block.  Replayed on the host, that must give exactly the image
    ``pack_weight`` builds from the 16-bit weight (ragged rows / K, two GLU sections)."""
    import torch
    from rhinoforge_b200.ops.kernels import pack_weight
    g = torch.Generator().manual_seed(0)
    for rows, K, sections in ((200, 150, 1), (256, 64, 2), (130, 200, 2)):
        q = torch.randint(-127, 128, (rows, K), generator=g, dtype=torch.int8)
        want = pack_weight(q.to(torch.float16), sections).view(torch.uint8)
        src = pack_weight(q, sections).view(torch.uint8)
        blocks = src.numel() // 8192
        assert want.numel() == blocks * 16384
        got = torch.zeros(blocks * 16384, dtype=torch.uint8)
        s8 = src.view(blocks, 128, 8, 8).view(torch.int8)                    # [block, row, piece, 8 values]
        wide = s8.to(torch.float16).view(torch.uint8).view(blocks, 128, 8, 16)   # 16 bytes per piece
        out = got.view(blocks, 128, 8, 16)
        r = torch.arange(128)[:, None]
        c = torch.arange(8)[None, :]
        pos = (c ^ (r & 7))                                                   # physical chunk of logical piece c in row r
        out[:, r.expand(128, 8), pos] = wide[:, r.expand(128, 8), c.expand(128, 8)]
        assert torch.equal(got, want.view(-1))


def test_persistent_tile_order_visits_every_tile_once_in_bands():
    """Host mirror of the persistent GEMM's tile order (bands of row tiles, rows fastest inside a band): a permutation
    of all tiles for any band size, with the short last band handled."""
    def coords(tile, tiles_m, tiles_n, band):
        per_band = band * tiles_n
        b, r = divmod(tile, per_band)
        rows_here = min(band, tiles_m - b * band)
        return b * band + r % rows_here, r // rows_here

    for tiles_m, tiles_n, band in ((64, 16, 16), (20, 8, 16), (7, 3, 2), (5, 5, 1), (9, 4, 100), (33, 5, 8)):
        band = min(band, tiles_m)
        seen = [coords(t, tiles_m, tiles_n, band) for t in range(tiles_m * tiles_n)]
        assert sorted(seen) == [(m, n) for m in range(tiles_m) for n in range(tiles_n)], (tiles_m, tiles_n, band)
        # consecutive tiles of a full band walk down the rows of one weight panel
        if tiles_m >= 2 * band:
            assert [c[0] for c in seen[:band]] == list(range(band)) and len({c[1] for c in seen[:band]}) == 1


def test_gemm_planner_invariants_over_decode_prefill_and_tensor_parallel_shapes():
    """Host-only launch plans (148 SMs assumed without a GPU): splits are powers of two and never exceed the k blocks,
    grids stay within two CTAs per SM times the cluster size for weight-streaming shapes, shared memory fits, two-shot
    all-reduce shapes do not split, big shapes go to the persistent kernel, and the all-reduce flag budget holds for every
    Qwen3-8B shard shape at TP 1/2/4/8."""
    import ctypes as C
    from rhinoforge_b200 import _native as N
    lib = N.lib()
    names = "swap bn splits stages gx gy smem kb ps twoshot".split()

    def plan(M, Nn, K, dual=False, int8=False, ar=0):
        g = N.RfGemm()
        g.M, g.N, g.K, g.dtype, g.force_swap, g.w_packed = M, Nn, K, 0, -1, 1
        g.x = g.w = g.out = 4096
        g.ldx, g.ldw, g.ldo = K, K, Nn
        if dual:
            g.dual_offset, g.act = Nn, 1
        if int8:
            g.w_int8, g.scale = 1, 4096
        if ar:
            g.ar_world, g.ar_rank, g.ar_recv, g.ar_flags, g.ar_state = ar, 0, 4096, 4096, 4096
            g.ar_recv_bytes, g.ar_flag_count = 1 << 40, (1 << 20) - 64
        out = (C.c_int32 * 10)()
        assert lib.rf_gemm_plan_info(C.byref(g), out) == 0, (M, Nn, K, lib.rf_last_error())
        return dict(zip(names, out))

    H = 4096
    for tp in (1, 2, 4, 8):
        I, QD, AD = 12288 // tp, 48 * 128 // tp, 32 * 128 // tp
        ar = tp if tp > 1 else 0
        for M in (1, 8, 64, 256):
            for (Nn, K, dual, a) in ((QD, H, False, 0), (H, AD, False, ar), (I, H, True, 0), (H, I, False, ar)):
                for int8 in (False, True):
                    p = plan(M, Nn, K, dual, int8, a)
                    S = p["splits"]
                    assert p["swap"] == 1 and S in (1, 2, 4, 8) and S <= p["kb"] and p["stages"] >= 2
                    assert p["gx"] * p["gy"] * S <= 2 * 148 or S == 1
                    assert p["smem"] <= 227 * 1024
                    if a:
                        assert p["gx"] * p["gy"] * 8 * a <= ((1 << 20) - 64) // 2
        for M in (2048, 8192):
            for (Nn, K, dual, a) in ((QD, H, False, 0), (H, AD, False, ar), (I, H, True, 0), (H, I, False, ar)):
                p = plan(M, Nn, K, dual, False, a)
                assert p["swap"] == 0 and p["smem"] <= 227 * 1024 and p["stages"] >= 2
                if a:
                    assert p["twoshot"] == 1 and p["splits"] == 1 and p["ps"] == 0
                    assert p["gx"] * p["gy"] * 8 * a <= ((1 << 20) - 64) // 2
                elif p["gx"] * p["gy"] >= 148:
                    assert p["ps"] == 1
    # the W8A16 gate/up decode shape fits two CTAs per SM
    p = plan(64, 12288, 4096, True, True)
    assert p["smem"] <= (228 * 1024 - 2048) // 2 and p["stages"] == 2 and p["splits"] == 2
    # short K: one k block per split is allowed
    assert plan(64, 4096, 512)["splits"] == 8 and plan(64, 4096, 128)["splits"] == 2


def test_bench_clock_sampler_reports_the_timed_region_only():
    """The sampler parses nvidia-smi CSV lines, reports samples taken after mark() (falling back to the last warm-up
    samples when the region is shorter than two sampling periods) and collects the throttle reasons it saw."""
    import importlib.util
    from pathlib import Path
    spec = importlib.util.spec_from_file_location("bench_mod", Path(__file__).resolve().parents[1] / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    class Done:
        def terminate(self): pass
        def wait(self, timeout=None): return 0

    def sampler(lines, first):
        s = bench.ClockSampler(0)
        s.proc, s.lines, s.first = Done(), list(lines), first
        return s.stop()

    idle = "0, 345, 1965, 140.2, 0x0000000000000001, Not Active, Not Active, Not Active, Not Active"
    busy = "0, 1965, 1965, 960.5, 0x0000000000000004, Not Active, Not Active, Not Active, Active"
    hot = "0, 1500, 1965, 990.0, 0x0000000000000040, Not Active, Active, Not Active, Active"
    r = sampler([idle, idle, busy, busy, busy], first=2)
    assert r["sm_mhz"] == 1965.0 and r["sm_max_mhz"] == 1965.0 and r["samples"] == 3 and r["reasons"] == ["sw_power_cap"]
    r = sampler([idle, busy, busy, busy, hot], first=4)          # one sample in the region: the warm-up tail is included
    assert r["samples"] == 5 and "hw_thermal_slowdown" in r["reasons"]
    r = sampler(["garbage", busy], first=0)
    assert r["samples"] == 1


# ----------------------------------------------------------------------------- install-completeness guard
def test_lazy_init_guard_finds_missing_declared_state():
    import torch.nn as nn
    from rhinoforge_b200.graph import (DynamoUnsafeLazyStateError, UninitializedLazyStateError, freeze_for_dynamo,
                                       mark_install_checked, verify_lazy_init)
    from rhinoforge_b200.graph.lazy_init_guard import missing_state, verify_graph_module_best_effort

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = nn.Linear(4, 4)

    model = nn.Sequential(Block(), Block(), nn.ReLU())
    verify_lazy_init(model)                                          # nobody opted in: nothing to check
    mark_install_checked(model[0], ("_rpu_handle_x",))
    model[1]._rpu_dynamo_safe = True                                 # the older marker spelling
    model[1]._rpu_required_attrs = ("_rpu_cos_sin", "proj")
    assert missing_state(model) == [("0", "Block", ["_rpu_handle_x"]), ("1", "Block", ["_rpu_cos_sin"])]
    with pytest.raises(UninitializedLazyStateError, match=r"0 \(Block\): missing \['_rpu_handle_x'\]"):
        verify_lazy_init(model)
    assert DynamoUnsafeLazyStateError is UninitializedLazyStateError and freeze_for_dynamo is verify_lazy_init
    model[0]._rpu_handle_x = object()
    model[1]._rpu_cos_sin = None                                     # present, even if None
    verify_lazy_init(model)
    mark_install_checked(model[0], ("_rpu_handle_x", "_rpu_other"))  # extends, no duplicates
    assert model[0]._rpu_required_attrs == ("_rpu_handle_x", "_rpu_other")
    with pytest.raises(UninitializedLazyStateError):
        verify_graph_module_best_effort(model)                       # walks direct children
    verify_graph_module_best_effort(object())                        # nothing with _modules: no-op

    class Handle:                                                    # runtime handles are not nn.Modules
        pass
    h = mark_install_checked(Handle(), ("engine",))
    with pytest.raises(UninitializedLazyStateError, match="<root>"):
        verify_lazy_init(h)
    h.engine = 1
    verify_lazy_init(h)


def test_guard_marker_names_are_known_runtime_attributes():
    from rhinoforge_b200.runtime import hw_attrs
    for name in ("_rpu_lazy_init_checked", "_rpu_dynamo_safe", "_rpu_required_attrs"):
        assert hw_attrs.classify(name) == "internal"


# ----------------------------------------------------------------------------- adapter template
def test_adapter_template_refuses_until_filled_then_behaves_like_a_family(monkeypatch):
    from types import SimpleNamespace
    import torch
    from rhinoforge_b200.adapters._template import MinimalCausalLMAdapter, TemplateNotFilledError, register
    from rhinoforge_b200.api.errors import UnsupportedModelError
    from rhinoforge_b200.runtime import live_handle, registry

    cfg = SimpleNamespace(model_type="llama", hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                          num_attention_heads=2, num_key_value_heads=1, head_dim=64, vocab_size=64, rms_norm_eps=1e-5,
                          rope_theta=1e4, tie_word_embeddings=True)
    with pytest.raises(TemplateNotFilledError, match="ARCH, FAMILY, SUPPORTED_PROFILES"):
        MinimalCausalLMAdapter.preflight(cfg)
    with pytest.raises(TemplateNotFilledError):
        register()

    class TinyAdapter(MinimalCausalLMAdapter):
        ARCH, FAMILY = "TinyForCausalLM", "Tiny"
        SUPPORTED_PROFILES = frozenset({(128, 256, 2, 1)})
        RENAMES = (("transformer.h.", "model.layers."), ("transformer.wte.", "model.embed_tokens."))

    TinyAdapter.preflight(cfg)
    with pytest.raises(UnsupportedModelError, match="deny by default"):
        TinyAdapter.preflight(SimpleNamespace(**{**vars(cfg), "hidden_size": 256}))
    with pytest.raises(UnsupportedModelError, match="head_dim"):
        TinyAdapter.preflight(SimpleNamespace(**{**vars(cfg), "head_dim": 80}))

    sd = {"transformer.wte.weight": torch.zeros(64, 128), "transformer.h.0.self_attn.q_proj.weight": torch.ones(128, 128),
          "model.norm.weight": torch.ones(128)}
    get_raw = lambda n: sd[n]
    get_raw.names = frozenset(sd)
    ad = TinyAdapter(config=cfg, get_weight=get_raw, rpu_execution={"prefill": {"chunk_size": 64}})
    try:
        dc = ad.decoder_config()
        assert (dc.hidden_size, dc.num_layers, dc.num_kv_heads, dc.qk_norm, dc.tie_embeddings) == (128, 2, 1, False, True)
        get = ad._weights()
        assert get("model.layers.0.self_attn.q_proj.weight").sum() == 128 * 128
        assert get("model.embed_tokens.weight").shape == (64, 128) and get("model.norm.weight").shape == (128,)
        assert "model.layers.0.self_attn.q_proj.weight" in get.names and "transformer.wte.weight" not in get.names
        ad._validate_shapes(dc, get)                                # the names the engine asks for are all present
        with pytest.raises(ValueError, match="not supported"):
            TinyAdapter(config=cfg, get_weight=get_raw, rpu_execution={"vision": {"chunk_size": 64}})
    finally:
        live_handle.release(ad) if hasattr(live_handle, "release") else None

    monkeypatch.setattr(registry, "ADAPTERS", dict(registry.ADAPTERS))
    register(TinyAdapter)
    assert registry.get_adapter("TinyForCausalLM") is TinyAdapter


# ----------------------------------------------------------------------------- compatibility report
def test_compatibility_report_classifies_linears_and_plans_their_decode_gemm(caplog):
    import logging
    import torch.nn as nn
    from rhinoforge_b200 import _native
    from rhinoforge_b200.runtime.weights import check_model_rpu_compatible, print_rpu_compatibility_report

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = nn.Linear(4096, 4096, bias=False)
            self.o_proj = nn.Linear(4096, 4096, bias=False)
            self.gate = nn.Linear(4096, 12288, bias=False)
            self.head = nn.Linear(100, 6, bias=False)            # 6 outputs split over 2 ranks at most
            self.odd = nn.Linear(37, 5, bias=False)              # splits nowhere; 74-byte rows are not TMA-aligned

    with torch.device("meta"):
        model = Block()
    info = check_model_rpu_compatible(model)
    assert (info["q_proj"]["status"], info["o_proj"]["status"], info["gate"]["status"]) == ("col", "row", "col")
    assert info["q_proj"]["tp"] == 8 and info["q_proj"]["shard"] == (512, 4096)
    assert info["o_proj"]["shard"] == (4096, 512) and info["gate"]["shard"] == (1536, 4096)
    assert info["head"]["status"] == "fallback" and info["head"]["tp"] == 2 and info["head"]["shard"] == (3, 100)
    assert info["odd"]["status"] == "fallback" and info["odd"]["tp"] == 1 and not info["odd"]["tma_ok"]
    assert "decode_plan" not in info["odd"]
    if _native.available():
        plan = info["o_proj"]["decode_plan"]                      # the tensor-parallel o_proj shard: short K, split fully
        assert plan["swap"] == 1 and plan["k_blocks"] == 8 and plan["splits"] == 8
        assert info["q_proj"]["decode_plan"]["swap"] == 1
    one = check_model_rpu_compatible(model, tp_degrees=(1,))
    assert one["head"]["status"] == "col" and one["head"]["shard"] == (6, 100)
    logger = logging.getLogger("rpu_backend")
    old_level, old_propagate = logger.level, logger.propagate
    logger.setLevel(logging.INFO)
    logger.propagate = True
    try:
        with caplog.at_level(logging.INFO, logger="rpu_backend"):
            print_rpu_compatibility_report(model)
    finally:
        logger.setLevel(old_level)
        logger.propagate = old_propagate
    text = caplog.text
    assert "5 Linear layers (accelerated: 3, col: 2, row: 1, fallback: 2)" in text
    assert "odd [5 x 37]: K rows are not 16-byte aligned" in text and "head [6 x 100]: no aligned" in text


# ----------------------------------------------------------------------------- Dynamo front-end
def test_partitioner_cuts_at_host_nodes_and_preserves_results():
    import torch.fx
    from rhinoforge_b200.graph.dynamo_partitioner import default_is_capturable, partition_for_capture

    class M(torch.nn.Module):
        def forward(self, x, w):
            y = torch.relu(x @ w)
            rows = y.sum(1).nonzero()                     # data-dependent shape: the host has to look
            z = y * 2 + rows.shape[0]
            return z, y.to("cpu"), z.to(torch.float64)    # a host copy is cut out, a dtype cast is not

    gm = torch.fx.symbolic_trace(M())
    parts = partition_for_capture(gm)
    assert [s.capturable for s in parts.segments] == [True, False, True, False, True]
    assert [s.n_nodes for s in parts.segments if not s.capturable] == [1, 1]
    x, w = torch.randn(4, 8), torch.randn(8, 8)
    got, want = parts.run((x, w)), M()(x, w)
    assert all(torch.equal(a, b) for a, b in zip(got, want))
    seen = []
    parts.run((x, w), lambda i, seg, fn, args: (seen.append((i, seg.capturable)), fn(*args))[1])
    assert seen == [(0, True), (1, False), (2, True), (3, False), (4, True)]
    names = {n.name: default_is_capturable(n) for n in gm.graph.nodes}
    assert not names["nonzero"] and names["relu"] and not names["to"] and names["to_1"]

    class Pure(torch.nn.Module):
        def forward(self, x):
            return torch.tanh(x) * 3
    one = partition_for_capture(torch.fx.symbolic_trace(Pure()))
    assert [s.capturable for s in one.segments] == [True] and torch.equal(one.run((x,)), torch.tanh(x) * 3)
    everything_host = partition_for_capture(torch.fx.symbolic_trace(Pure()), lambda n: False)
    assert [s.capturable for s in everything_host.segments] == [False]


def test_dynamo_backend_records_once_replays_after_and_bounds_its_table():
    from rhinoforge_b200.graph.dynamo_backend import RpuDynamoBackend, dynamo_backend
    from rhinoforge_b200.graph.lazy_init_guard import UninitializedLazyStateError, mark_install_checked
    torch._dynamo.reset()
    be = RpuDynamoBackend(max_entries=1)
    w = torch.randn(8, 8)

    @torch.compile(backend=be)
    def f(x):
        return torch.relu(x @ w) + 1

    x = torch.randn(4, 8)
    for _ in range(3):
        out = f(x)
    assert torch.allclose(out, torch.relu(x @ w) + 1)
    s = be.stats()
    assert (s["graphs"], s["records"], s["replays"], s["evictions"], s["entries"]) == (1, 1, 2, 0, 1)
    f(torch.randn(6, 8))                                    # another shape: re-trace, new signature, the old entry goes
    s = be.stats()
    assert s["records"] == 2 and s["evictions"] == 1 and s["entries"] == 1
    be.clear()
    assert be.stats()["entries"] == 0
    with pytest.raises(ValueError, match="max_entries"):
        RpuDynamoBackend(max_entries=0)
    assert isinstance(dynamo_backend, RpuDynamoBackend)

    # a module that still creates state in forward is refused when its graph reaches the backend
    class Lazy(torch.nn.Module):
        def forward(self, x):
            return x + 1
    lazy = mark_install_checked(Lazy(), ("_rpu_table",))
    holder = torch.nn.Module()
    holder.child = lazy
    with pytest.raises(UninitializedLazyStateError):
        be(holder, ())
    torch._dynamo.reset()


def test_action_denormalizer_config_constructors_and_unapply(tmp_path):
    import json
    import numpy as np
    from rhinoforge_b200.api.action_denorm import EPS, ActionDenormalizer, ActionGroup
    stats = {"norm_stats": {"action.arm.position": {"mean": [1.0, 2.0, 3.0], "std": [0.5, 0.5, 2.0]},
                            "action.gripper": {"min": [0.0], "max": [0.08], "mean": [0.04], "std": [0.01]},
                            "observation.state.arm.position": {"mean": [0.0] * 3, "std": [1.0] * 3}}}
    path = tmp_path / "norm.json"
    path.write_text(json.dumps(stats))
    train = {"data": {"joints": ["{'arm.position': 3}", {"gripper": 1}],
                      "norm_type": ["{'arm.position': 'meanstd'}", "{'gripper': 'minmax'}"]}}
    robot = {"actions": [{"action.arm.position": {"subtract_state": True}}, {"action.gripper": {"subtract_state": False}}]}
    d = ActionDenormalizer.from_training_config(str(path), train, robot_config=robot)
    assert [(g.key, g.dim, g.norm_type, g.subtract_state) for g in d.groups] == [
        ("action.arm.position", 3, "meanstd", True), ("action.gripper", 1, "minmax", False)]
    assert d.groups[0].state_key == "observation.state.arm.position" and d.real_dim == 4
    a = torch.tensor([[[0.0, 1.0, -1.0, 0.0, 9.0, 9.0], [2.0, 0.0, 0.0, 5.0, 9.0, 9.0]]])     # [1, H, padded D]
    state = [10.0, 20.0, 30.0, 99.0]
    out = d.unapply(a, state)
    assert out.dtype == torch.float32 and out.shape == (2, 4)
    want_arm0 = np.array([0.0, 1.0, -1.0]) * (np.array([0.5, 0.5, 2.0]) + EPS) + [1, 2, 3] + np.array(state[:3])
    assert np.allclose(out[0, :3].numpy(), want_arm0, atol=1e-5)
    assert abs(float(out[0, 3]) - 0.04) < 1e-5 and abs(float(out[1, 3]) - 0.24) < 1e-5      # 5.0 is not clipped: (5+1)/2*0.08
    # the reference's own example: x=[1.5,-2.0], min=[0,0], max=[2,4] -> [2.5,-2.0]; minmax == minmax_woclip on the way back
    for kind in ("minmax", "minmax_woclip"):
        mm = ActionDenormalizer([ActionGroup("g", 2, kind)], {"g": {"min": np.zeros(2), "max": np.array([2.0, 4.0])}})
        assert np.allclose(mm.unapply([[1.5, -2.0]]).numpy(), [[2.5, -2.0]], atol=1e-5)
    # per-step [chunk, dim] statistics are cut to the action horizon; a shorter table is refused
    per_step = {"g": {"mean": np.arange(8.0).reshape(4, 2), "std": np.ones((4, 2))}}
    ps = ActionDenormalizer([ActionGroup("g", 2, "meanstd")], per_step)
    assert np.allclose(ps.unapply(np.zeros((3, 2))).numpy(), np.arange(6.0).reshape(3, 2), atol=1e-5)
    with pytest.raises(ValueError, match="horizon 4 < action horizon 5"):
        ps.unapply(np.zeros((5, 2)))
    with pytest.raises(ValueError, match="non-finite statistics"):
        ActionDenormalizer([ActionGroup("g", 2, "std")], {"g": {"std": np.array([1.0, np.inf])}})
    with pytest.raises(ValueError, match="empty horizon"):
        ActionDenormalizer([ActionGroup("g", 2, "std")], {"g": {"std": np.zeros((0, 2))}})
    with pytest.raises(ValueError, match="no state was provided"):
        d.unapply(a)
    with pytest.raises(ValueError, match="state has 2 dims"):
        d.unapply(a, [1.0, 2.0])
    with pytest.raises(ValueError, match="non-finite"):
        d.unapply(torch.tensor([[float("nan"), 0, 0, 0]]), state)
    with pytest.raises(ValueError, match="non-finite"):
        d.unapply(a, [float("inf"), 0, 0, 0])
    with pytest.raises(ValueError, match="expected batch 1"):
        d.unapply(torch.zeros(2, 3, 4), state)
    with pytest.raises(ValueError, match="< real_dim 4"):
        d.unapply(torch.zeros(3, 2), state)
    absolute = ActionDenormalizer.from_training_config(str(path), train["data"])             # no robot config: absolute
    assert not any(g.subtract_state for g in absolute.groups)
    assert np.allclose(absolute.unapply(a)[0, :3].numpy(), want_arm0 - np.array(state[:3]), atol=1e-5)
    with pytest.raises(ValueError, match=r"missing explicit norm_type entries for action groups \['gripper'\]"):
        ActionDenormalizer.from_training_config(str(path), {"joints": train["data"]["joints"],
                                                            "norm_type": ["{'arm.position': 'meanstd'}"]})

    auto = ActionDenormalizer.from_norm_json(str(path), robot_config=robot)
    assert [(g.key, g.dim, g.norm_type) for g in auto.groups] == [("action.arm.position", 3, "meanstd"),
                                                                  ("action.gripper", 1, "meanstd")]
    assert auto.groups[0].subtract_state and auto.groups[1].state_key == "observation.state.gripper"
    only_state = tmp_path / "state_only.json"
    only_state.write_text(json.dumps({"observation.state.x": {"mean": [0.0], "std": [1.0]}}))
    with pytest.raises(ValueError, match="no 'action.\\*' keys"):
        ActionDenormalizer.from_norm_json(str(only_state))
    spec = ActionDenormalizer.from_spec(str(path), [ActionGroup("action.gripper", 1, "minmax")])
    assert abs(float(spec.unapply([[-1.0]])[0, 0])) < 1e-6

    yaml_path = tmp_path / "train.yaml"
    yaml_path.write_text("data:\n  joints:\n    - \"{'arm.position': 3}\"\n  norm_type:\n    - \"{'arm.position': 'std'}\"\n")
    from_yaml = ActionDenormalizer.from_training_config(str(path), str(yaml_path))
    assert from_yaml.groups[0].norm_type == "std" and from_yaml.real_dim == 3


def test_mrope_table_builders_match_the_hugging_face_formulations():
    """Interleaved (Qwen3-VL) and chunked (Qwen2.5-VL) M-RoPE, stated the way the Hugging Face modules compute them."""
    from rhinoforge_b200.runtime.rope_partial import build_chunked_mrope_cos_sin, build_interleaved_mrope_cos_sin
    hd, theta, section = 128, 1e6, [24, 20, 20]
    g = torch.Generator().manual_seed(0)
    pos = torch.randint(0, 500, (37, 3), generator=g)
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    freqs = pos.t().double()[:, :, None] * inv[None, None, :]                        # [3, seq, half]
    # Qwen3-VL apply_interleaved_mrope: start from T, overwrite slice(offset, section*3, 3) with H / W
    inter = freqs[0].clone()
    for dim, off in ((1, 1), (2, 2)):
        idx = slice(off, section[dim] * 3, 3)
        inter[:, idx] = freqs[dim][:, idx]
    cos, sin = build_interleaved_mrope_cos_sin(pos, head_dim=hd, rope_theta=theta, mrope_section=section)
    assert cos.dtype == sin.dtype == torch.float16 and cos.shape == (37, 64) and cos.device.type == "cpu"
    assert torch.equal(cos, inter.cos().half()) and torch.equal(sin, inter.sin().half())
    # Qwen2.5-VL: split the frequency axis by section, take chunk i from axis i % 3
    chunks = torch.cat([part[i % 3] for i, part in enumerate(freqs.split(section, dim=-1))], dim=-1)
    cos_c, sin_c = build_chunked_mrope_cos_sin(pos, head_dim=hd, rope_theta=theta, mrope_section=section)
    assert torch.equal(cos_c, chunks.cos().half()) and torch.equal(sin_c, chunks.sin().half())
    assert not torch.equal(cos, cos_c)
    # partial rotary: tables cover rotary_dim only
    part, _ = build_interleaved_mrope_cos_sin(pos, head_dim=256, rope_theta=theta, mrope_section=[11, 11, 10], rotary_dim=64)
    assert part.shape == (37, 32)
    text_only = torch.arange(9)[:, None].expand(9, 3).contiguous()                   # equal axes: plain 1-D RoPE
    c1, _ = build_interleaved_mrope_cos_sin(text_only, head_dim=hd, rope_theta=theta, mrope_section=section)
    assert torch.equal(c1, (torch.arange(9).double()[:, None] * inv[None]).cos().half())
    for kw, exc in ((dict(mrope_section=[24, 20, 19]), ValueError), (dict(rotary_dim=130), ValueError),
                    (dict(rotary_dim=63), ValueError), (dict(rope_theta=0.0), ValueError)):
        with pytest.raises(exc):
            build_interleaved_mrope_cos_sin(pos, **{**dict(head_dim=hd, rope_theta=theta, mrope_section=section), **kw})
    with pytest.raises(ValueError, match=r"\[seq, 3\]"):
        build_chunked_mrope_cos_sin(pos.t(), head_dim=hd, rope_theta=theta, mrope_section=section)
    with pytest.raises(TypeError, match="integer"):
        build_chunked_mrope_cos_sin(pos.float(), head_dim=hd, rope_theta=theta, mrope_section=section)


def test_hw_attr_validator_over_a_module_tree():
    import torch.nn as nn
    from rhinoforge_b200.runtime import hw_attrs as H
    from rhinoforge_b200.runtime.errors import RPUConfigError

    def tree():
        return nn.Sequential(nn.Linear(4, 4), nn.Sequential(nn.Linear(4, 4), nn.ReLU()))

    m = tree()
    m._rpu_execution = {"prefill": {"chunk_size": 64}}           # a user may set this ahead of the install
    m[0]._rpu_debug_tag = "first"
    H.validate_preinstall(m)
    m[1][0]._rpu_handle = 7                                      # runtime-owned: stale before an install
    with pytest.raises(RPUConfigError, match="'_rpu_handle' on Linear before the install"):
        H.validate_preinstall(m)
    H.validate_postinstall(m)                                    # ... but legitimate after one
    m[1]._rpu_chunksize = 64                                     # a typo
    with pytest.raises(RPUConfigError, match="'_rpu_chunksize' on Sequential after the install"):
        H.validate_existing_hw_attrs(m)
    with pytest.raises(RPUConfigError):
        H.install_hw_attr_validator(m)                           # scanned first: nothing was stamped
    assert type(m) is nn.Sequential and type(m[0]) is nn.Linear
    del m[1]._rpu_chunksize

    H.install_hw_attr_validator(m)
    H.install_hw_attr_validator(m)                               # idempotent
    assert type(m).__name__ == "Validated_Sequential" and type(m[0]).__name__ == "Validated_Linear"
    assert isinstance(m[0], nn.Linear) and type(m[0]) is type(m[1][0])       # one cached subclass per class
    assert m(torch.zeros(2, 4)).shape == (2, 4)                  # forward is untouched
    m[0]._rpu_dtype = torch.float16                              # cold names can still be set before the first forward
    m[0]._rpu_is_ready = True                                    # so can runtime-owned ones
    with pytest.raises(RPUConfigError, match="not a known runtime attribute"):
        m[1][1]._rpu_typo = 1
    m[0].some_user_field = 3                                     # foreign names are nobody's business

    H.mark_first_forward_done(m)
    m[0]._rpu_dtype = torch.float16                              # same value: fine
    with pytest.raises(RPUConfigError, match="cannot change afterwards"):
        m[0]._rpu_dtype = torch.bfloat16
    with pytest.raises(RPUConfigError, match="owned by the runtime"):
        m[1][0]._rpu_handle = 8
    m[1][1]._rpu_debug_tag = "hot"                               # public names stay writable
    other = tree()
    H.install_hw_attr_validator(other)
    other[0]._rpu_dtype = torch.bfloat16                         # another tree has its own state
    H.mark_first_forward_done(object())                          # never stamped: no-op
    H.mark_first_forward_done(3)

    class Slotted:
        __slots__ = ("x",)
    with pytest.raises(RPUConfigError, match="does not allow the validator"):
        H.install_hw_attr_validator(Slotted())                   # a class whose layout forbids the swap is reported


def test_runtime_handle_opts_into_the_install_check():
    from types import SimpleNamespace
    from rhinoforge_b200.graph.lazy_init_guard import verify_lazy_init
    from rhinoforge_b200.runtime.causal_lm import RPUCausalLM
    engine = SimpleNamespace(dtype=torch.float16, tp=SimpleNamespace(world=1), device=torch.device("cpu"))
    handle = RPUCausalLM(engine, SimpleNamespace(), execution={"prefill": {"chunk_size": 64}})
    assert handle._rpu_lazy_init_checked and set(handle._rpu_required_attrs) >= {"engine", "_rpu_execution", "_rpu_dtype"}
    verify_lazy_init(handle)
    del handle._rpu_dtype
    with pytest.raises(RuntimeError, match="_rpu_dtype"):
        verify_lazy_init(handle)
