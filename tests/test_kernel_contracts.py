"""Source contracts of the native layer and of the adapters (no GPU, no weights)."""
import re
from pathlib import Path
from types import SimpleNamespace

import pytest

ROOT = Path(__file__).resolve().parents[1]
CSRC = ROOT / "rhinoforge_b200" / "csrc"
SOURCES = [p for p in CSRC.rglob("*") if p.suffix in (".cu", ".cuh", ".cpp", ".h")]


def _text(p: Path) -> str:
    return p.read_text(encoding="utf-8")


def test_every_kernel_launch_goes_through_the_counted_launcher():
    """No raw triple-chevron launches: launch_k adds the programmatic-dependent-launch attribute and
    every launch is counted (the bench reports the number)."""
    for p in SOURCES:
        assert "<<<" not in _text(p), f"{p.name} has a raw kernel launch"


def test_no_forbidden_cuda_entry_points_or_cluster_multicast_loads():
    """The batched-memcpy entry points and cluster-multicast loads stay out of the tree.  The patterns are
    assembled from pieces so that this file does not itself contain them."""
    batched = "Memcpy" + "Batch" + "Async"
    batched3d = "Memcpy3D" + "Batch" + "Async"
    mcast = ".multi" + "cast::" + "cluster"
    for p in SOURCES + list((ROOT / "rhinoforge_b200").rglob("*.py")):
        t = _text(p)
        assert batched not in t and batched3d not in t, f"{p} names a batched memcpy entry point"
        loads = [ln for ln in t.splitlines() if mcast in ln and "tcgen05.commit" not in ln and not ln.lstrip().startswith("//")]
        assert not loads, f"{p} has a cluster-multicast load: {loads[:1]}"


def test_device_waits_are_bounded():
    """Every spin on an mbarrier or a peer flag is one of the helpers in ptx.cuh, which give up after a time limit."""
    ptx = _text(CSRC / "common" / "ptx.cuh")
    assert "globaltimer" in ptx
    for helper in ("bool mbar_wait(", "bool wait_flag_ge_sys("):
        i = ptx.index(helper)
        body = ptx[i:ptx.index("\n}\n", i)]
        assert "limit_ns" in body and "return false" in body and "global_timer_ns" in body, f"{helper} has no time limit"
    for p in SOURCES:
        if p.name == "ptx.cuh":
            continue
        t = _text(p)
        assert "try_wait" not in t, f"{p.name} spins on an mbarrier outside the bounded helper"
        assert "ld.acquire.sys" not in t, f"{p.name} polls peer memory outside the bounded helper"


def test_waiting_kernels_report_and_release():
    """Kernels that can time out record a status and still reach the TMEM release at the end."""
    g = _text(CSRC / "kernels" / "gemm_tc.cu")
    assert g.count("report_status") >= 5
    assert g.rindex("tmem_dealloc") > g.rindex("report_status")
    # the only early exit allowed is the shared-memory alignment check, which runs before anything is acquired
    kernel = g[g.index("gemm_tc_kernel("):g.index("// ------------------------------------------------------------ host side")]
    assert "return;" not in kernel[kernel.index("tmem_alloc("):], "an early return after the TMEM allocation leaks it"
    assert kernel[:kernel.index("tmem_alloc(")].count("return;") <= 1


def test_qwen3_5_geometry_guard_fires_from_the_config_alone():
    from rhinoforge_b200.adapters.qwen3_5 import Qwen3_5Adapter
    from rhinoforge_b200.runtime.errors import UnsupportedModelError
    cfg = SimpleNamespace(model_type="qwen3_5_text", vocab_size=1000, hidden_size=1024, intermediate_size=3584,
                          num_hidden_layers=24, num_attention_heads=8, num_key_value_heads=2, head_dim=256,
                          rms_norm_eps=1e-6, layer_types=["linear_attention"] * 18 + ["full_attention"] * 6,
                          linear_num_key_heads=16, linear_num_value_heads=16, linear_key_head_dim=96,
                          linear_value_head_dim=128, linear_conv_kernel_dim=4, max_position_embeddings=4096,
                          rope_parameters={"rope_theta": 1e7, "partial_rotary_factor": 0.25, "mrope_section": [11, 11, 10]})
    with pytest.raises(UnsupportedModelError, match="Dk=96"):
        Qwen3_5Adapter.preflight(cfg)
    cfg.linear_key_head_dim = 128
    Qwen3_5Adapter.preflight(cfg)                           # admitted 0.8B profile
    cfg.num_experts = 64
    with pytest.raises(UnsupportedModelError, match="mixture-of-experts"):
        Qwen3_5Adapter.preflight(cfg)


def test_examples_preflight_before_loading_weights():
    for name, guard, load in (("dinov3.py", "DINOv3Adapter.preflight(", "AutoModel.from_pretrained("),
                              ("qwen3_5_text.py", "Qwen3_5Adapter.preflight(", "AutoModelForCausalLM.from_pretrained(")):
        t = _text(ROOT / "examples" / name)
        assert t.index(guard) < t.index(load), f"{name} loads weights before the config-only preflight"


def test_pi05_variant_gate_and_policy_constructor_contract():
    from rhinoforge_b200.adapters.pi05 import config_from_policy_config
    from rhinoforge_b200.api.policy import Pi05Policy
    from rhinoforge_b200.runtime.errors import UnsupportedModelError
    with pytest.raises(UnsupportedModelError, match="variant pair"):
        config_from_policy_config({"paligemma_variant": "gemma_2b", "action_expert_variant": "gemma_2b"})
    with pytest.raises(RuntimeError, match="not a public constructor"):
        Pi05Policy()
    with pytest.raises(ValueError, match="trust_remote_code=False"):
        Pi05Policy.from_pretrained("/nonexistent", trust_remote_code=True)
