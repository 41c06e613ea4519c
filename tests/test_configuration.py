"""Configuration tiers: rpu_execution validation, portable TOML files, --check-config without torch,
runner environment policy, documentation <-> source inventory of environment variables."""
from __future__ import annotations

import os
import pickle
import re
import subprocess
import sys
import tomllib
from pathlib import Path

import pytest

from rpu_backend.api._execution import bind_rpu_execution, normalize_rpu_execution

ROOT = Path(__file__).resolve().parents[1]


def test_execution_configuration_is_validated_and_frozen():
    cfg = normalize_rpu_execution({"prefill": {"chunk_size": 128, "padding_budget": 64}}, entry_point="test",
                                  supported={"prefill": ("chunk_size", "padding_budget")})
    assert dict(cfg["prefill"]) == {"chunk_size": 128, "padding_budget": 64}
    with pytest.raises(TypeError, match="read-only"):
        cfg["prefill"].chunk_size = 64
    with pytest.raises(ValueError, match="positive multiple of 16"):
        normalize_rpu_execution({"prefill": {"chunk_size": 17}}, entry_point="test")
    with pytest.raises(ValueError, match="conflicts"):
        normalize_rpu_execution({"prefill": {"padding_rows": 16, "padding_budget": 16}}, entry_point="test")
    with pytest.raises(ValueError, match="unknown stage"):
        normalize_rpu_execution({"decode": {}}, entry_point="test")
    with pytest.raises(ValueError, match="unknown field"):
        normalize_rpu_execution({"prefill": {"tile": 1}}, entry_point="test")
    with pytest.raises(TypeError, match="must be a mapping"):
        normalize_rpu_execution([], entry_point="test")
    assert normalize_rpu_execution(None, entry_point="t", vlm_chunk_size=0)["prefill"]["chunk_size"] == "auto"
    import copy
    assert copy.deepcopy(cfg) is cfg and pickle.loads(pickle.dumps(cfg)) == cfg


def test_execution_binding_is_cold():
    class Owner:
        pass
    o = Owner()
    first = bind_rpu_execution(o, {"prefill": {"chunk_size": 64}}, entry_point="t")
    assert bind_rpu_execution(o, {"prefill": {"chunk_size": 64}}, entry_point="t") is first
    assert bind_rpu_execution(o, None, entry_point="t") is first
    with pytest.raises(ValueError, match="conflicts with the existing"):
        bind_rpu_execution(o, {"prefill": {"chunk_size": 128}}, entry_point="t")


def test_example_toml_files_are_portable():
    configs = sorted((ROOT / "examples" / "configs").glob("*.toml"))
    assert configs
    banned = ("/nfs", "/data/", "10.10.", "192.168.", "hf_", "token=", "/root/")
    for p in configs:
        text = p.read_text(encoding="utf-8")
        assert tomllib.loads(text)
        assert not any(b in text for b in banned), p


def test_model_example_check_config_does_not_import_native(tmp_path):
    guard = tmp_path / "guard"
    for pkg in ("rpu_backend", "rhinoforge_b200"):
        (guard / pkg).mkdir(parents=True)
        (guard / pkg / "__init__.py").write_text(f"raise AssertionError('{pkg} imported')\n")
    (guard / "torch.py").write_text("raise AssertionError('torch imported')\n")
    env = {**os.environ, "PYTHONPATH": str(guard)}
    scripts = sorted(p for p in (ROOT / "examples").glob("*.py")
                     if p.name not in ("verify_install.py", "_config.py"))
    assert scripts
    for s in scripts:
        r = subprocess.run([sys.executable, "-S", str(s), "--check-config"], cwd=ROOT, env=env, text=True,
                           capture_output=True, timeout=30)
        assert r.returncode == 0, (s.name, r.stdout, r.stderr)
        assert "configuration OK" in r.stdout


@pytest.mark.parametrize("body,expected", [
    ("[runner.env]\nRPU_NOT_A_DOCUMENTED_OPTION = 1", "not documented"),
    ("[runner.env]\nRPU_KERNEL_LIB_PATH = 'x'", "not allowed"),
    ("[runner.env]\nRPU_API_TOKEN = 'x'", "not allowed"),
    ("[runner.env]\nLD_PRELOAD = 'x'", "not documented"),
    ("[runner.env]\nRF_TP_REPORT = 'x'", "diagnostic-only"),
    ("[rpu_execution.vision]\nchunk_size = 256", "not supported by this model entry point"),
    ("[runner.torch_profile]\nenabled = 'yes'", "must be a boolean"),
    ("[runner.hw_profile]\nmax_dumps = 0", "positive integer"),
])
def test_full_runner_rejects_unsafe_configuration(tmp_path, body, expected):
    cfg = tmp_path / "invalid.toml"
    cfg.write_text('[runner]\ntarget = "causal_lm"\n' + body + '\n[model]\nalias = "qwen3-0.6b"\n'
                   '[generation]\nprompt = "hi"\nmax_new_tokens = 4\n')
    r = subprocess.run([sys.executable, str(ROOT / "examples" / "run_model.py"), "--config", str(cfg),
                        "--check-config"], cwd=ROOT, text=True, capture_output=True, timeout=60)
    assert r.returncode != 0
    assert expected in r.stderr


def test_runner_applies_environment_only_for_execution(tmp_path, monkeypatch):
    sys.path.insert(0, str(ROOT / "examples"))
    try:
        import importlib
        run_model = importlib.import_module("run_model")
    finally:
        sys.path.pop(0)
    cfg = run_model.load_config(ROOT / "examples" / "configs" / "qwen3_0_6b_full.toml")
    assert cfg.target == "causal_lm" and cfg.env == {"RPU_LOG_LEVEL": 3, "RPU_WARMUP": 1}
    monkeypatch.delenv("RPU_WARMUP", raising=False)
    run_model.run_target(cfg.target, cfg.path, check_config=True)      # --check-config path
    assert "RPU_WARMUP" not in os.environ
    run_model.apply_environment({"RPU_WARMUP": 1, "RPU_SKIP_IDLE_RECORD_FUNCTION": True})
    assert os.environ["RPU_WARMUP"] == "1" and os.environ["RPU_SKIP_IDLE_RECORD_FUNCTION"] == "1"
    monkeypatch.delenv("RPU_WARMUP")
    monkeypatch.delenv("RPU_SKIP_IDLE_RECORD_FUNCTION")


def test_environment_inventory_matches_sources():
    """Every variable the Python sources read is documented, and every documented project variable is read."""
    doc = (ROOT / "docs" / "runtime_config.md").read_text()
    documented = set(re.findall(r"^\| `([A-Z][A-Z0-9_]+)` \|", doc, re.MULTILINE))
    dropped = {"RPU_KERNEL_LIB_PATH", "LKN_MAX_BATCH_ENTRIES", "LKN_KD_BUF_MB", "LKN_INSTR_BUF_MB"}
    pattern = re.compile(r"[\"']((?:RPU|RF|QWEN3|LKN)_[A-Z0-9_]+)[\"']")
    used = set()
    files = list((ROOT / "rhinoforge_b200").rglob("*.py")) + [ROOT / "bench.py"]
    files += list((ROOT / "rhinoforge_b200" / "csrc").rglob("*.cpp")) + list((ROOT / "rhinoforge_b200" / "csrc").rglob("*.cu"))
    for f in files:
        used |= set(pattern.findall(f.read_text(encoding="utf-8")))
    used |= {"RF_TP_REPORT", "RF_DEBUG_BOUNDS"}          # read by the test workers / the build script
    used -= dropped
    project_documented = {n for n in documented if not n.startswith(("HF_", "HUGGINGFACE_"))}
    assert used - documented == set(), f"undocumented: {sorted(used - documented)}"
    assert project_documented - used == set(), f"documented but unused: {sorted(project_documented - used)}"
    for d in dropped:
        assert f"`{d}`" in doc


def test_rhinovla_example_runs_the_whole_lifecycle_with_its_stand_in_factory(tmp_path):
    """construct -> prepare graphs -> predict, with the execution handshake, on a machine without a GPU; a request that
    the runtime cannot honour is reported by the policy, not swallowed."""
    script = ROOT / "examples" / "rhinovla.py"
    r = subprocess.run([sys.executable, str(script)], cwd=ROOT, text=True, capture_output=True, timeout=300)
    assert r.returncode == 0, (r.stdout, r.stderr)
    assert "shape=(32, 7)" in r.stdout and "'chunk_size': 256" in r.stdout and "'execution_alignment': 16" in r.stdout
    bad = tmp_path / "vision.toml"
    bad.write_text((ROOT / "examples" / "configs" / "rhinovla.toml").read_text().replace(
        "[rpu_execution.action]", "[rpu_execution.vision]"))
    r = subprocess.run([sys.executable, str(script), "--config", str(bad)], cwd=ROOT, text=True, capture_output=True, timeout=300)
    assert r.returncode != 0 and "not supported by this model entry point" in r.stderr


def test_version_comes_from_the_project_table():
    import rhinoforge_b200
    from rhinoforge_b200._version import API_VERSION, DISTRIBUTION_VERSION
    project = tomllib.loads((ROOT / "pyproject.toml").read_text(encoding="utf-8"))["project"]
    assert DISTRIBUTION_VERSION == project["version"] == rhinoforge_b200.__version__
    assert API_VERSION.split(".")[0] == "5"
