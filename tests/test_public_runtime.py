"""Host-only contract of the public package surface (no GPU needed)."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_host_only_import_is_silent():
    site = [p for p in sys.path if "site-packages" in p]
    script = (f"import sys; sys.path.insert(0, {str(ROOT)!r}); sys.path.extend({site!r}); "
              "import rpu_backend, torch; assert rpu_backend.__version__; assert hasattr(torch, 'rpu'); "
              "import rhinoforge_b200; assert rhinoforge_b200.RPUCache is rpu_backend.RPUCache")
    env = os.environ.copy()
    env.pop("PYTHONPATH", None)
    env["CUDA_VISIBLE_DEVICES"] = ""
    r = subprocess.run([sys.executable, "-S", "-c", script], cwd=ROOT, env=env, text=True, capture_output=True)
    assert r.returncode == 0, r.stderr
    assert r.stdout == "" and r.stderr == ""


def test_nofile_preflight_is_silent_and_best_effort(monkeypatch, capsys):
    from rpu_backend import _bootstrap_env
    calls = []
    monkeypatch.setattr(_bootstrap_env.resource, "getrlimit", lambda _k: (1024, 4096))
    monkeypatch.setattr(_bootstrap_env.resource, "setrlimit", lambda k, v: calls.append((k, v)))
    _bootstrap_env.ensure_nofile_limit()
    assert calls == [(_bootstrap_env.resource.RLIMIT_NOFILE, (4096, 4096))]

    def deny(*_a):
        raise OSError("denied")
    monkeypatch.setattr(_bootstrap_env.resource, "setrlimit", deny)
    _bootstrap_env.ensure_nofile_limit()
    out = capsys.readouterr()
    assert out.out == out.err == ""


def test_public_api_and_host_graph_lifecycle():
    import torch
    import rpu_backend
    from rpu_backend.graph import GraphCache, GraphSignature
    assert rpu_backend.__all__ == ["__version__", "RPUCache", "RPUModelForCausalLM", "reset_graph_cache"]
    assert sorted(dir(rpu_backend)) == sorted(rpu_backend.__all__)
    if torch.cuda.is_available():
        pytest.skip("host-only lifecycle is checked without a device")
    cache = GraphCache()
    sig = GraphSignature(op_id="host-contract", shapes=(1, 16))
    assert cache.phase == "CONFIGURING" and cache.size() == 0 and cache.cache_invariant_ok()
    cache.begin_warmup()
    with cache.capture(sig):
        pass
    assert cache.phase == "WARMING"
    with pytest.raises(RuntimeError, match=r"requires the C\+\+ backend"):
        cache.freeze()
    assert cache.explain_miss(sig).startswith("miss at GmId")


def test_removed_names_point_to_replacements():
    import rpu_backend
    with pytest.raises(AttributeError, match="RPUCache.from_model"):
        rpu_backend.build_rpu_cache
    with pytest.warns(DeprecationWarning):
        assert rpu_backend.GraphCache is rpu_backend.graph.GraphCache


def test_external_adapter_registration():
    from rpu_backend.runtime import registry

    class PublicTestAdapter:
        pass

    arch = "RhinoForgePublicTestArchitecture"
    try:
        registry.register_adapter(arch, PublicTestAdapter)
        assert registry.get_adapter(arch) is PublicTestAdapter
        assert arch in registry.list_adapters()
        registry.register_adapter(arch, PublicTestAdapter)
        with pytest.raises(RuntimeError, match="already registered"):
            registry.register_adapter(arch, type("OtherAdapter", (), {}))
    finally:
        registry.ADAPTERS.pop(arch, None)


def test_plugins_cannot_shadow_builtins():
    from rpu_backend.runtime import registry
    api = registry._plugin_api(frozenset(registry.ADAPTERS))
    with pytest.raises(RuntimeError, match="built-in"):
        api.register_adapter("Qwen3ForCausalLM", type("Shadow", (), {}))
    from rpu_backend.api.errors import UnsupportedModelError
    with pytest.raises(UnsupportedModelError):
        registry.get_adapter("NoSuchArchitectureForCausalLM")


def test_builtin_adapters_load_lazily():
    r = subprocess.run([sys.executable, "-c",
                        "import sys; import rpu_backend; "
                        "assert not any(m.startswith('rhinoforge_b200.adapters.qwen3') for m in sys.modules); "
                        "from rpu_backend.runtime.registry import get_adapter; "
                        "c = get_adapter('Qwen3ForCausalLM'); assert c.__name__ == 'Qwen3Adapter'"],
                       cwd=ROOT, text=True, capture_output=True, env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0, r.stderr


def test_registry_excludes_unsupported_profiles():
    from rpu_backend import model_registry
    required = {"qwen3-0.6b", "llama-3.2-1b", "qwen3-vl-2b", "qwen3-vl-4b", "qwen3_5-0.8b", "dinov3-vit-b",
                "pi05-libero-finetuned", "qwen3-14b-w8a16-lmhead-int8"}
    excluded = {"qwen3-vl-8b", "dinov3-vit-s", "dinov3-vit-l", "gemma2", "paligemma2", "lingbot-vla-4b", "qwen3-14b",
                "qwen3-0.6b-w8a16-lmhead-int8", "qwen3-8b-w8a16-lmhead-int8", "qwen3-0.6b-instruct"}
    assert required <= model_registry.MODELS.keys()
    assert excluded.isdisjoint(model_registry.MODELS)
    for rel in model_registry.MODELS.values():
        p = Path(rel)
        assert not p.is_absolute() and ".." not in p.parts
    with pytest.raises(KeyError, match="Unknown model"):
        model_registry.model_path("nope")


def test_model_cache_override(monkeypatch, tmp_path):
    from rpu_backend import model_registry
    monkeypatch.setenv("RPU_MODEL_CACHE", str(tmp_path))
    monkeypatch.delenv("HF_HOME", raising=False)
    assert model_registry.model_path("qwen3-0.6b") == tmp_path / "Qwen3-0.6B"
    assert model_registry.hf_cache_root() == tmp_path / ".hf"


def test_error_hierarchy():
    from rpu_backend.api import errors as E
    for name in ("RPUConfigError", "UnsupportedModelError", "RPUUnsupportedDtypeError", "RPUSingleHandleError",
                 "SPMExhaustionError", "WeightShapeMismatchError"):
        assert issubclass(getattr(E, name), E.RPUBackendError)


def test_strict_boolean_env_parser(monkeypatch):
    from rpu_backend.runtime.control import rpu_env_bool, rpu_env_exact1
    monkeypatch.delenv("RPU_TEST_FLAG", raising=False)
    assert rpu_env_bool("RPU_TEST_FLAG", True) is True
    for raw, want in ((" On ", True), ("1", True), ("false", False), ("", False), ("0", False)):
        monkeypatch.setenv("RPU_TEST_FLAG", raw)
        assert rpu_env_bool("RPU_TEST_FLAG") is want
    monkeypatch.setenv("RPU_TEST_FLAG", "yes")
    with pytest.raises(ValueError, match="must be one of"):
        rpu_env_bool("RPU_TEST_FLAG")
    assert rpu_env_exact1("RPU_TEST_FLAG") is False
    monkeypatch.setenv("RPU_TEST_FLAG", "1")
    assert rpu_env_exact1("RPU_TEST_FLAG") is True


def test_native_struct_layouts_match_ctypes():
    """The ctypes mirrors must have the C sizes, or every kernel argument would be misread."""
    import ctypes as C
    from rhinoforge_b200 import _native as N
    if not N.available():
        pytest.skip("native library not built")
    lib = N.lib()
    sizes = (C.c_int32 * 16)()
    lib.rf_struct_sizes(sizes)
    got = [C.sizeof(t) for t in (N.RfGemm, N.RfRopeKv, N.RfAttn, N.RfStackConfig, N.RfLayerWeights, N.RfStackComm,
                                 N.RfStackForward)]
    assert list(sizes)[:7] == got
    assert list(sizes)[8:11] == [C.sizeof(N.RfConv1d), C.sizeof(N.RfGdn), C.sizeof(N.RfArConsume)]


def test_torch_ops_rpu_namespace_is_registered_and_runs_on_cpu():
    """The stand-alone operators exist by name; on CPU tensors they take the plain PyTorch path."""
    import torch
    import rhinoforge_b200  # noqa: F401
    ops = torch.ops.rpu
    for name in ("rms_norm", "apply_rotary_pos_emb", "scaled_dot_product_attention_unified", "gather_embedding",
                 "assemble_inputs_embeds", "cast_uint8_fp16", "linear_into", "lm_head_logits_top1", "argmax_lastdim_host",
                 "moe_select", "reset_graph_cache"):
        assert hasattr(ops, name), name
    x = torch.randn(3, 8)
    y = ops.rms_norm(x, torch.ones(8), 1e-6)
    assert torch.allclose(y, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-5)
    q = torch.randn(2, 5, 4, 16)
    kv = torch.randn(2, 5, 2, 16)
    o = ops.scaled_dot_product_attention_unified(q, kv, kv, True, 0.0)
    assert o.shape == q.shape
    ids, w = ops.moe_select(torch.randn(4, 8), None, 2, 1.0)
    assert ids.shape == (4, 2) and torch.allclose(w.sum(-1), torch.ones(4), atol=1e-5)
    assert torch.equal(ops.argmax_lastdim_host(torch.tensor([[1.0, 3.0, 2.0]])), torch.tensor([1], dtype=torch.int32))


def test_handle_family_ops_exist_and_keep_their_books_on_cpu():
    """Every in-scope handle family has create / set_weights / forward / destroy under ``torch.ops.rpu``; handles are
    typed (a vision handle is refused by a decoder op), destroyed handles are gone, forward before weights fails."""
    import json
    import pytest
    import torch
    import rhinoforge_b200  # noqa: F401
    from rhinoforge_b200.ops import handle_ops
    from rhinoforge_b200.runtime.errors import RPUBackendError, RPUConfigError
    ops = torch.ops.rpu
    for fam in handle_ops.FAMILIES:
        for suffix in ("create", "set_weights", "forward", "destroy"):
            assert hasattr(ops, f"{fam}_{suffix}"), f"{fam}_{suffix}"
    for name in ("causal_decoder_set_weights_w8a16", "qwen3_5_set_weights_w8a16", "pi05_denoise_loop_forward",
                 "assemble_inputs_embeds_rev", "cast_uint8_fp16_into", "conv2d_mc_nhwc", "spm_alloc_init",
                 "spm_alloc_reset_temporary", "spm_alloc_reset_all", "spm_alloc_dump"):
        assert hasattr(ops, name), name
    h = ops.siglip_create(json.dumps({"hidden_size": 64}))
    d = ops.causal_decoder_create("{}")
    assert handle_ops.live_handles()[h] == "siglip" and handle_ops.live_handles()[d] == "causal_decoder"
    with pytest.raises(RPUBackendError, match="belongs to family"):
        ops.causal_decoder_destroy(h)
    with pytest.raises(RPUBackendError, match="no weights yet"):
        ops.siglip_forward(h, torch.zeros(1, 3, 8, 8))
    with pytest.raises(RPUConfigError):
        ops.pi05_create("{not json")
    ops.siglip_destroy(h)
    ops.causal_decoder_destroy(d)
    assert h not in handle_ops.live_handles() and d not in handle_ops.live_handles()
    with pytest.raises(RPUBackendError, match="unknown or destroyed"):
        ops.siglip_destroy(h)
    # stand-alone additions on CPU tensors
    x = torch.randn(2, 4, 4, 8)
    w = torch.randn(6, 8, 2, 2)
    y = ops.conv2d_mc_nhwc(x, w, None, 2, 0)
    ref = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2), w, stride=2).permute(0, 2, 3, 1)
    assert torch.allclose(y, ref, atol=1e-5)
    e = torch.randn(5, 3)
    assert torch.equal(ops.assemble_inputs_embeds_rev(e, torch.tensor([4, 0])), e[[4, 0]])
    out = torch.empty(2, 2, dtype=torch.float16)
    ops.cast_uint8_fp16_into(torch.tensor([[0, 255], [1, 2]], dtype=torch.uint8), out, 1.0 / 255.0, 0.0)
    assert abs(float(out[0, 1]) - 1.0) < 1e-3
    ops.spm_alloc_init(); ops.spm_alloc_reset_temporary(); ops.spm_alloc_reset_all()
    assert json.loads(ops.spm_alloc_dump())["initialised"] is True


def test_standalone_ops_propagate_shapes_on_meta_and_fake_tensors():
    """Shape-only implementations: the operators trace on ``device='meta'`` and under ``FakeTensorMode`` with fake CUDA
    tensors (no GPU, no data pointers)."""
    import torch
    import rhinoforge_b200  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    ops = torch.ops.rpu
    m = lambda *s, dtype=torch.float16: torch.empty(*s, device="meta", dtype=dtype)
    assert ops.rms_norm(m(3, 8), m(8), 1e-6).shape == (3, 8)
    assert ops.gather_embedding(m(100, 16), m(2, 5, dtype=torch.int64)).shape == (2, 5, 16)
    assert ops.assemble_inputs_embeds_rev(m(9, 4), m(3, dtype=torch.int64)).shape == (3, 4)
    assert ops.cast_uint8_fp16(m(2, 3, dtype=torch.uint8), 1.0, 0.0).dtype == torch.float16
    assert ops.conv2d_mc_nhwc(m(1, 28, 28, 3), m(16, 3, 14, 14), None, 14, 0).shape == (1, 2, 2, 16)
    assert ops.lm_head_logits_top1(m(4, 8), m(32, 8)).shape == (4,)
    ids, w = ops.moe_select(m(4, 8), None, 2, 1.0)
    assert ids.dtype == torch.int32 and w.dtype == torch.float32 and ids.shape == w.shape == (4, 2)
    with FakeTensorMode():
        a = torch.empty(7, 16, device="cuda", dtype=torch.float16)
        y = ops.rms_norm(a, torch.empty(16, device="cuda", dtype=torch.float16), 1e-6)
        q = torch.empty(2, 5, 4, 16, device="cuda", dtype=torch.float16)
        kv = torch.empty(2, 5, 2, 16, device="cuda", dtype=torch.float16)
        o = ops.scaled_dot_product_attention_unified(q, kv, kv, True, 0.0)
    assert y.shape == (7, 16) and y.device.type == "cuda" and o.shape == q.shape


def test_handle_forward_ops_propagate_shapes_from_the_handle_config():
    """A handle's configuration is host data, so ``*_forward`` can be shape-traced with fake tensors; the grid-driven
    towers, whose length depends on tensor values, refuse instead of guessing."""
    import json
    import logging
    import torch
    import rhinoforge_b200  # noqa: F401
    from rhinoforge_b200.runtime.errors import RPUBackendError
    from torch._subclasses.fake_tensor import FakeTensorMode
    ops = torch.ops.rpu
    made = {"causal_decoder": ops.causal_decoder_create(json.dumps({"vocab_size": 1000, "hidden_size": 64,
                                                                   "torch_dtype": "bfloat16"})),
            "siglip": ops.siglip_create(json.dumps({"hidden_size": 96, "patch_size": 14, "image_size": 224})),
            "hyvit2": ops.hyvit2_create(json.dumps({"hidden_size": 96, "patch_size": 16, "image_size": 64,
                                                    "rpu_projector_dim": 40})),
            "dinov3_vision": ops.dinov3_vision_create(json.dumps({"hidden_size": 64, "patch_size": 16})),
            "pi05": ops.pi05_create("{}"), "qwen3vl_vision": ops.qwen3vl_vision_create("{}")}
    try:
        cu = lambda *s, dtype=torch.float16: torch.empty(*s, device="cuda", dtype=dtype)
        with FakeTensorMode():
            logits = ops.causal_decoder_forward(made["causal_decoder"], cu(2, 5, 64, dtype=torch.bfloat16), [], [], None, 0,
                                                True, None, None, None, None)
            sig, = ops.siglip_forward(made["siglip"], cu(3, 3, 224, 224))
            hy, = ops.hyvit2_forward(made["hyvit2"], cu(1, 3, 64, 64))
            tokens, cls = ops.dinov3_vision_forward(made["dinov3_vision"], cu(1, 3, 224, 224))
            img, msk, tok = cu(2, 3, 3, 224, 224), cu(2, 3), cu(2, 48, dtype=torch.int64)
            act = ops.pi05_forward(made["pi05"], img, msk, tok, cu(2, 48), cu(2, 50, 32, dtype=torch.float32))
            lens = ops.gemma_forward(made["pi05"], img, msk, tok, cu(2, 48))
            step = ops.pi05_denoise_loop_forward(made["pi05"], None, cu(2, 50, 32), 10)
            logging.disable(logging.ERROR)                           # torch logs the refusal before re-raising it
            try:
                with pytest.raises(RPUBackendError, match="data-dependent output length"):
                    ops.qwen3vl_vision_forward(made["qwen3vl_vision"], cu(16, 1536), cu(1, 3, dtype=torch.int64))
            finally:
                logging.disable(logging.NOTSET)
        assert (tuple(logits.shape), logits.dtype, logits.device.type) == ((2, 1000), torch.bfloat16, "cuda")
        assert tuple(sig.shape) == (3, 256, 96) and tuple(hy.shape) == (1, 16, 40)
        assert tuple(tokens.shape) == (1, 1 + 4 + 196, 64) and tuple(cls.shape) == (1, 64)
        assert tuple(act.shape) == (2, 50, 32) and act.dtype == torch.float16 and tuple(step.shape) == (2, 50, 32)
        assert tuple(lens.shape) == (2,) and lens.dtype == torch.int32
        on_meta = ops.causal_decoder_forward(made["causal_decoder"], torch.empty(5, 64, device="meta"), [], [], None, 0, True,
                                             None, None, None, None)
        assert tuple(on_meta.shape) == (1, 1000)
        with pytest.raises(RPUBackendError, match="belongs to family"):
            ops.siglip_forward(made["pi05"], torch.empty(1, 3, 224, 224, device="meta"))
    finally:
        for fam, h in made.items():
            getattr(ops, fam + "_destroy")(h)


def test_handle_ops_build_model_configs_from_json():
    """The JSON a ``*_create`` op receives becomes the runtime's config object: nested Pi0.5 geometry, dtype names."""
    import torch
    from rhinoforge_b200.ops import handle_ops as H
    c = H._pi05_config({"action_dim": 7, "horizon": 16, "num_views": 2,
                        "vlm": {"hidden": 128, "inter": 256, "layers": 2, "heads": 2, "kv_heads": 1, "head_dim": 64},
                        "expert": {"hidden": 64, "inter": 128, "layers": 2, "heads": 2, "kv_heads": 1, "head_dim": 64},
                        "vision": {"hidden_size": 128, "intermediate_size": 256, "num_hidden_layers": 2,
                                   "num_attention_heads": 2, "image_size": 56, "patch_size": 14}})
    assert (c.action_dim, c.horizon, c.num_views, c.vlm.hidden, c.expert.inter, c.vision.patch_size) == (7, 16, 2, 128, 128, 14)
    assert c.tokens_per_image == 16
    d = H._pi05_config({})
    assert (d.vlm.hidden, d.expert.hidden, d.horizon) == (2048, 1024, 50)
    assert H._dtype_of({"torch_dtype": "bfloat16"}) == torch.bfloat16 and H._dtype_of({}) == torch.float16
    assert H._dtype_of({"dtype": "torch.float16"}) == torch.float16


def test_torch_rpu_controls_and_debug_surface(tmp_path):
    """Setters are reflected by their getters; fixed properties of the design answer as documented; the probe-tensor
    store and the trace configuration can be inspected and cleared."""
    import torch
    import rhinoforge_b200  # noqa: F401
    r = torch.rpu
    assert r.get_ddr_flush() is False
    r.set_ddr_flush(True)
    assert r.get_ddr_flush() is True
    r.set_ddr_flush(False)
    assert r.get_ddr_flush_force() is True and r.get_spm_mode() is False
    assert r.get_linear_acc32() is True and r.get_allreduce_twostage() is True and r.is_autocast_available() is True
    assert r.get_amp_supported_dtype() == [torch.float16, torch.bfloat16]
    before = r.get_cross_layer_batch_size()
    r.set_cross_layer_batch_prefill(4)
    assert r.get_cross_layer_batch_prefill() == r.get_cross_layer_batch_size() == 4
    r.set_cross_layer_batch_size(before)
    with pytest.raises(ValueError):
        r.set_cross_layer_batch_size(-1)
    assert set(r.get_memory_stats()) == {"allocated_bytes", "reserved_bytes", "peak_allocated_bytes"}
    assert r.get_memory_stats() == r.memory_stats()
    r.reset_peak_memory_stats(); r.reset_accumulated_memory_stats()          # no device: no-ops
    r.reset_temporary_spm(); r.spm_alloc_reset_temporary(); r.reset_all_spm()
    assert r.is_available() == (torch.cuda.is_available() and rhinoforge_b200._native.available())

    from rhinoforge_b200.runtime import debug
    r.set_debug_export(True)
    try:
        debug.export_debug_tensor("layer0.attn_out", torch.arange(4.0))
        debug.export_debug_tensor("layer0.mlp_out", torch.ones(2))
        assert r.list_debug_tensors() == ["layer0.attn_out", "layer0.mlp_out"]
        assert torch.equal(r.get_debug_tensor("layer0.attn_out"), torch.arange(4.0))
        r.clear_debug_tensors()
        assert r.list_debug_tensors() == [] and r.get_debug_tensor("layer0.attn_out") is None
    finally:
        r.set_debug_export(False)
    assert r.get_spm_debug() is False
    r.set_spm_debug(True)
    assert r.get_spm_debug() is True
    r.set_spm_debug(False)
    assert r.get_hw_perf_trace()["dir"] is None
    r.set_hw_perf_trace(str(tmp_path / "trace"), 3)
    assert r.get_hw_perf_trace() == {"dir": str(tmp_path / "trace"), "max_dumps": 3, "seq": 0}
    r.set_hw_perf_trace(None, 0)
    assert r.get_hw_perf_trace()["dir"] is None
