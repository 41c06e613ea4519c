#!/usr/bin/env python3
"""Full runner: one TOML file owns the model request, the runtime environment and profiling.

    python examples/run_model.py --config examples/configs/qwen3_0_6b_full.toml [--check-config]

``[runner] target`` picks the example script; ``[runner.env]`` variables are validated against the
inventory in ``docs/runtime_config.md`` (undocumented, credential-like, dropped and diagnostic-only
names are refused) and applied only for a real run, before torch or the backend is imported;
``[runner.torch_profile]`` wraps the run in ``torch.profiler`` (CPU + CUDA activities, Chrome trace),
``[runner.hw_profile]`` in ``torch.rpu.hw_perf_trace`` (per-scope kernel traces).
"""
from __future__ import annotations

import argparse
import contextlib
import os
import re
import runpy
import sys
import tomllib
from dataclasses import dataclass, field
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
HERE = Path(__file__).resolve().parent
DEFAULT_CONFIG = HERE / "configs" / "qwen3_0_6b_full.toml"

TARGETS = {name: f"{name}.py" for name in
           ("causal_lm", "dinov3", "hy_embodied", "pi05", "qwen3_5_text", "qwen3_vl", "rhinovla", "wall_oss")}
_PREFILL = ("chunk_size", "padding_rows", "padding_budget")
EXECUTION_SUPPORT = {
    "causal_lm": {"prefill": _PREFILL},
    "dinov3": {"vision": ("chunk_size",)},
    "hy_embodied": {},
    "pi05": {"prefill": _PREFILL, "vision": ("chunk_size",), "action": ("chunk_size",)},
    "qwen3_5_text": {"prefill": _PREFILL},
    "qwen3_vl": {"prefill": _PREFILL, "vision": ("chunk_size",)},
    "rhinovla": None,
    "wall_oss": {"prefill": _PREFILL, "vision": ("chunk_size",), "action": ("chunk_size",)},
}
DENIED_ENV = {"RPU_KERNEL_LIB_PATH", "LKN_MAX_BATCH_ENTRIES", "LKN_KD_BUF_MB", "LKN_INSTR_BUF_MB"}
CREDENTIAL_MARKERS = ("TOKEN", "SECRET", "PASSWORD", "CREDENTIAL", "API_KEY")


@dataclass
class ProfileSettings:
    torch_enabled: bool = False
    torch_output: str = "profiles/torch_trace.json"
    record_shapes: bool = False
    profile_memory: bool = False
    with_stack: bool = False
    hw_enabled: bool = False
    hw_output_dir: str = "profiles/hw"
    hw_max_dumps: int = 32


@dataclass
class RunnerConfig:
    path: Path
    target: str
    env: dict = field(default_factory=dict)
    profile: ProfileSettings = field(default_factory=ProfileSettings)
    raw: dict = field(default_factory=dict)


def env_inventory() -> tuple[set, set]:
    """(documented names, diagnostic-only names) parsed from the tables of docs/runtime_config.md."""
    text = (ROOT / "docs" / "runtime_config.md").read_text(encoding="utf-8")
    diag_head, ctl_head = "## Diagnostic-only inventory", "## Non-environment runtime controls"
    if diag_head not in text or ctl_head not in text:
        raise RuntimeError("docs/runtime_config.md is missing its inventory headings")
    row = re.compile(r"^\| `([A-Z][A-Z0-9_]+)` \|", re.MULTILINE)
    diag = text.split(diag_head, 1)[1].split(ctl_head, 1)[0]
    return set(row.findall(text)), set(row.findall(diag))


def _table(parent: dict, key: str, label: str, allowed: set) -> dict:
    t = parent.get(key, {})
    if not isinstance(t, dict):
        raise ValueError(f"{label} must be a table")
    extra = sorted(set(t) - allowed)
    if extra:
        raise ValueError(f"{label} has unsupported key(s): {', '.join(extra)}")
    return t


def _flag(t: dict, key: str, label: str) -> bool:
    v = t.get(key, False)
    if not isinstance(v, bool):
        raise ValueError(f"{label}.{key} must be a boolean")
    return v


def load_config(path: Path) -> RunnerConfig:
    with path.open("rb") as f:
        raw = tomllib.load(f)
    runner = raw.get("runner")
    if not isinstance(runner, dict):
        raise ValueError("configuration needs a [runner] table")
    extra = sorted(set(runner) - {"target", "env", "torch_profile", "hw_profile"})
    if extra:
        raise ValueError(f"[runner] has unsupported key(s): {', '.join(extra)}")
    target = runner.get("target")
    if target not in TARGETS:
        raise ValueError(f"[runner].target must be one of: {', '.join(sorted(TARGETS))}")
    if raw.get("rpu_execution") is not None:
        # the validator is a leaf module: load it by path so that nothing else is imported
        mod = runpy.run_path(str(ROOT / "rhinoforge_b200" / "api" / "_execution.py"))
        mod["normalize_rpu_execution"](raw["rpu_execution"], entry_point="examples/run_model.py",
                                       supported=EXECUTION_SUPPORT[target])
    env = runner.get("env", {})
    if not isinstance(env, dict):
        raise ValueError("[runner.env] must be a table")
    documented, diagnostic = env_inventory()
    for name, value in env.items():
        if name in DENIED_ENV or any(m in name for m in CREDENTIAL_MARKERS):
            raise ValueError(f"[runner.env].{name} is not allowed")
        if name not in documented:
            raise ValueError(f"[runner.env].{name} is not documented in docs/runtime_config.md")
        if name in diagnostic:
            raise ValueError(f"[runner.env].{name} is diagnostic-only and cannot be set in TOML")
        if not isinstance(value, (str, int, bool)):
            raise ValueError(f"[runner.env].{name} must be a string, integer, or boolean")
    tp = _table(runner, "torch_profile", "[runner.torch_profile]",
                {"enabled", "output", "record_shapes", "profile_memory", "with_stack"})
    hp = _table(runner, "hw_profile", "[runner.hw_profile]", {"enabled", "output_dir", "max_dumps"})
    prof = ProfileSettings(
        torch_enabled=_flag(tp, "enabled", "[runner.torch_profile]"),
        torch_output=tp.get("output", "profiles/torch_trace.json"),
        record_shapes=_flag(tp, "record_shapes", "[runner.torch_profile]"),
        profile_memory=_flag(tp, "profile_memory", "[runner.torch_profile]"),
        with_stack=_flag(tp, "with_stack", "[runner.torch_profile]"),
        hw_enabled=_flag(hp, "enabled", "[runner.hw_profile]"),
        hw_output_dir=hp.get("output_dir", "profiles/hw"), hw_max_dumps=hp.get("max_dumps", 32))
    if not isinstance(prof.torch_output, str) or not prof.torch_output:
        raise ValueError("[runner.torch_profile].output must be a path string")
    if not isinstance(prof.hw_output_dir, str) or not prof.hw_output_dir:
        raise ValueError("[runner.hw_profile].output_dir must be a path string")
    if not isinstance(prof.hw_max_dumps, int) or isinstance(prof.hw_max_dumps, bool) or prof.hw_max_dumps < 1:
        raise ValueError("[runner.hw_profile].max_dumps must be a positive integer")
    return RunnerConfig(path, target, dict(env), prof, raw)


def apply_environment(env: dict) -> None:
    for name, value in env.items():
        os.environ[name] = ("1" if value else "0") if isinstance(value, bool) else str(value)


def run_target(target: str, config_path: Path, *, check_config: bool) -> None:
    script = HERE / TARGETS[target]
    argv = [str(script), "--config", str(config_path)] + (["--check-config"] if check_config else [])
    saved = sys.argv
    try:
        sys.argv = argv
        runpy.run_path(str(script), run_name="__main__")
    except SystemExit as e:
        if e.code not in (None, 0):
            raise
    finally:
        sys.argv = saved


def run_profiled(cfg: RunnerConfig) -> None:
    p = cfg.profile
    profiler = None
    if p.torch_enabled or p.hw_enabled:
        import torch
    if p.torch_enabled:
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        profiler = torch.profiler.profile(activities=acts, record_shapes=p.record_shapes,
                                          profile_memory=p.profile_memory, with_stack=p.with_stack)
    try:
        with contextlib.ExitStack() as stack:
            if profiler is not None:
                stack.enter_context(profiler)
            if p.hw_enabled:
                sys.path.insert(0, str(ROOT))
                import rpu_backend  # noqa: F401  (installs torch.rpu)
                out = Path(p.hw_output_dir).expanduser()
                out.mkdir(parents=True, exist_ok=True)
                stack.enter_context(torch.rpu.hw_perf_trace(str(out), max_dumps=p.hw_max_dumps))
            run_target(cfg.target, cfg.path, check_config=False)
    finally:
        if profiler is not None:       # the trace is written even when the run raised
            out = Path(p.torch_output).expanduser()
            out.parent.mkdir(parents=True, exist_ok=True)
            profiler.export_chrome_trace(str(out))
            print(f"torch profile: {out}")


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", type=Path, default=DEFAULT_CONFIG)
    ap.add_argument("--check-config", action="store_true")
    ap.add_argument("--list-targets", action="store_true")
    a = ap.parse_args()
    if a.list_targets:
        print("\n".join(sorted(TARGETS)))
        return 0
    cfg = load_config(a.config.expanduser().resolve())
    if a.check_config:
        run_target(cfg.target, cfg.path, check_config=True)
        print(f"runner configuration OK: {cfg.path}")
        return 0
    apply_environment(cfg.env)
    run_profiled(cfg)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
