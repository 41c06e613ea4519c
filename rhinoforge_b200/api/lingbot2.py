"""``Lingbot2Policy``: public facade of the LingBot-VLA-v2 policy (Qwen3-VL prefix + sparse-MoE action expert).

    policy = Lingbot2Policy.from_checkpoint(ckpt_dir, robot_norm_path=..., training_config_path=...).to("rpu")
    policy.prepare_graphs(images=[...], instruction="...", proprioception=[...])   # optional: BUILD + check + freeze
    out = policy.infer(images=[...], instruction="...", proprioception=[...])      # Lingbot2ActionOutput
    out.actions            # [H, 16] physical units (needs the de-normalisation files)
    out.actions_normalized # [H, 16] in the model's normalised space;  out.actions_full: [H, 55];  out.latency_ms
    policy.close()

The checkpoint, the camera roster and the precision profile are fixed at construction; pixels, instruction and
proprioception change per call.  The model emits a NORMALISED ``[horizon, 55]`` grid of which the first 16 columns are
real degrees of freedom (dual arm 14 + effectors 2); physical units need the robot's normalisation statistics together
with the matching training configuration (the statistics alone cannot prove joint order or normalisation kind), or an
explicit ``action_norm_spec``.  ``obs=`` accepts an already pre-processed observation (``pixel_values``,
``image_grid_thw``, ``lang_tokens``, ``state``, ``noise``), which is also what lets the policy run without the
tokenizer / image processor files.

Reference: ``python/rpu_backend/api/lingbot2.py:357-1210``.
"""
from __future__ import annotations

import dataclasses
import json
import os
import threading
import time
from collections.abc import Mapping, Sequence
from typing import Any, Dict, Optional

import torch

from ._runtime_env import normalize_runtime_env
from .errors import RPUBackendError, RPUConfigError, UnsupportedModelError

VALID_ACTION_DIMS = 16
_RUNTIME_ENV_ALLOWLIST = frozenset({"RPU_LINGBOT2_DENOISE_UNROLL", "RPU_WARMUP"})
_DTYPES = ("fp16", "bf16")
_QUANT_PROFILES = ("w8a16", "w4a16")


@dataclasses.dataclass(frozen=True)
class Lingbot2ActionOutput:
    """One action chunk.  ``actions`` raises unless de-normalisation was configured: a normalised grid must never be
    consumed as physical units by accident."""

    actions_normalized: torch.Tensor
    actions_full: torch.Tensor
    latency_ms: float
    phase_ms: Dict[str, float]
    actions_physical: Optional[torch.Tensor] = None
    extra: Dict[str, Any] = dataclasses.field(default_factory=dict)

    @property
    def actions(self) -> torch.Tensor:
        if self.actions_physical is None:
            raise RPUBackendError(
                "LingBot-VLA-V2 actions are normalized, not physical-unit actions: build the policy with "
                "Lingbot2Policy.from_checkpoint(..., robot_norm_path=<robot norm-stats JSON>, "
                "training_config_path=<lingbotvla_cli.yaml>) to get de-normalized physical-unit actions. To inspect the "
                "normalized grid on purpose, read .actions_normalized / .actions_full instead.")
        return self.actions_physical

    @property
    def robot_ready(self) -> bool:
        """True iff a physical-unit de-normaliser was applied (not a certification of anything else)."""
        return self.actions_physical is not None


def _serialized(method):
    """One call into the policy at a time: the engine's graph inputs are shared static buffers."""
    def wrapped(self, *args, **kwargs):
        with self._lock:
            return method(self, *args, **kwargs)
    wrapped.__name__, wrapped.__doc__ = method.__name__, method.__doc__
    return wrapped


class Lingbot2Policy:
    def __init__(self) -> None:
        raise RuntimeError("Lingbot2Policy() is not a public constructor. Use "
                           "Lingbot2Policy.from_checkpoint(...).to('rpu').")

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_checkpoint(cls, ckpt_dir, *, dtype: str = "fp16", n_cameras: int = 3, image_size: int = 256,
                        max_lang_tokens: int = 72, robot_norm_path=None, training_config_path=None,
                        robot_config_path=None, action_norm_spec=None, runtime_env: Optional[Mapping] = None,
                        qwen3vl_base=None) -> "Lingbot2Policy":
        """Bind a policy to a checkpoint directory (``config.json`` + safetensors shards, optionally the Qwen3-VL
        processor files).  Nothing is read yet; ``.to('rpu')`` builds the runtime.  All argument errors are raised
        here, before any weight is touched."""
        dtype = (dtype or "fp16").strip().lower()
        if dtype in _QUANT_PROFILES:
            raise UnsupportedModelError(f"LingBot-VLA-V2 precision profile {dtype!r} is not built in this framework: the "
                                        "MoE expert bank runs in 16 bits (fp16 / bf16)")
        if dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(_DTYPES + _QUANT_PROFILES)}, got {dtype!r}")
        if isinstance(max_lang_tokens, bool) or not isinstance(max_lang_tokens, int):
            raise ValueError(f"max_lang_tokens must be a positive integer, got {max_lang_tokens!r}")
        if max_lang_tokens <= 0:
            raise ValueError(f"max_lang_tokens must be positive, got {max_lang_tokens}")
        if isinstance(n_cameras, bool) or not isinstance(n_cameras, int) or n_cameras <= 0:
            raise ValueError(f"n_cameras must be a positive integer, got {n_cameras!r}")
        self = object.__new__(cls)
        self._ckpt_dir = os.fspath(ckpt_dir)
        self._dtype = dtype
        self._n_cameras, self._image_size, self._max_lang_tokens = n_cameras, int(image_size), max_lang_tokens
        fs = lambda p: None if p is None else os.fspath(p)
        self._robot_norm_path, self._training_config_path = fs(robot_norm_path), fs(training_config_path)
        self._robot_config_path, self._action_norm_spec = fs(robot_config_path), action_norm_spec
        self._qwen3vl_base = fs(qwen3vl_base)
        self._runtime_env = normalize_runtime_env(runtime_env, owner="Lingbot2Policy", allowed=_RUNTIME_ENV_ALLOWLIST)
        self._engine = None
        self._processor = None
        self._denorm = None
        self._closed = False
        self._lock = threading.RLock()
        self._prepare_ms: Dict[str, float] = {}
        self._graph_profile: Optional[dict] = None
        self._one_graph = True
        return self

    @classmethod
    def _from_engine(cls, engine, *, denorm=None, max_lang_tokens: int = 72) -> "Lingbot2Policy":
        """A policy over an already built engine (tests, embedding applications that assemble the runtime themselves)."""
        self = object.__new__(cls)
        self._ckpt_dir, self._dtype = None, "fp16" if engine.dtype == torch.float16 else "bf16"
        self._n_cameras, self._image_size, self._max_lang_tokens = 0, 0, max_lang_tokens
        self._robot_norm_path = self._training_config_path = self._robot_config_path = self._action_norm_spec = None
        self._qwen3vl_base, self._runtime_env = None, {}
        self._engine, self._processor, self._denorm = engine, None, denorm
        self._closed = False
        self._lock = threading.RLock()
        self._prepare_ms, self._graph_profile = {}, None
        self._one_graph = True
        return self

    @property
    def dtype(self) -> str:
        return self._dtype

    @property
    def robot_ready(self) -> bool:
        return self._engine is not None and not self._closed and self._denorm is not None

    @property
    def graphs_ready(self) -> bool:
        return self._engine is not None and not self._closed and self._graph_profile is not None

    @property
    def graph_profile(self) -> Optional[dict]:
        return None if not self.graphs_ready else dict(self._graph_profile)

    # ------------------------------------------------------------------ build
    def _build_denormalizer(self):
        from .action_denorm import ActionDenormalizer
        if self._action_norm_spec is not None:
            if self._robot_norm_path is None:
                raise RPUConfigError("action_norm_spec needs robot_norm_path (the statistics file)")
            d = ActionDenormalizer.from_spec(self._robot_norm_path, list(self._action_norm_spec))
        elif self._robot_norm_path is not None:
            if self._training_config_path is None:
                raise RPUConfigError("robot_norm_path needs training_config_path: the statistics file alone cannot prove "
                                     "joint order or normalisation kinds")
            d = ActionDenormalizer.from_training_config(self._robot_norm_path, self._training_config_path,
                                                        robot_config=self._robot_config_path)
        else:
            return None
        if any(g.subtract_state for g in d.groups):
            raise RPUConfigError("delta (subtract_state) action groups are refused: the flat padded state input carries "
                                 "no metadata that proves joint-offset alignment")
        if d.real_dim != VALID_ACTION_DIMS:
            raise RPUConfigError(f"the action groups total {d.real_dim} dimensions, LingBot-VLA-V2 has {VALID_ACTION_DIMS}")
        return d

    @_serialized
    def to(self, device: Any) -> "Lingbot2Policy":
        from ..runtime.device import resolve_device
        if self._closed:
            raise RPUBackendError("Lingbot2Policy is closed")
        dev = resolve_device(device)
        if dev.type != "cuda":
            raise RPUBackendError(f"Lingbot2Policy runs on the accelerator only, got device {device!r}")
        if self._engine is not None:
            return self
        self._denorm = self._build_denormalizer()          # configuration errors first, before weights are read
        t0 = time.perf_counter()
        from ._loading import checkpoint_tensor_getter
        from ..adapters.lingbot_vla_v2 import build_engine
        with open(os.path.join(self._ckpt_dir, "config.json"), "r", encoding="utf-8") as f:
            config = json.load(f)
        get = checkpoint_tensor_getter(self._ckpt_dir)
        old_env = {k: os.environ.get(k) for k in self._runtime_env}
        os.environ.update(self._runtime_env)
        try:
            from ..runtime.control import rpu_env_bool
            self._one_graph = rpu_env_bool("RPU_LINGBOT2_DENOISE_UNROLL", True)     # 0: one launch sequence per Euler step
            self._engine = build_engine(config, get, device=dev, dtype=torch.float16 if self._dtype == "fp16" else torch.bfloat16,
                                        max_lang_tokens=self._max_lang_tokens, n_cameras=self._n_cameras,
                                        image_size=self._image_size, qwen3vl_base=self._qwen3vl_base)
        finally:
            for k, v in old_env.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
        self._prepare_ms["build_ms"] = (time.perf_counter() - t0) * 1000.0
        return self

    def _require_ready(self, what: str):
        if self._closed:
            raise RPUBackendError("Lingbot2Policy is closed")
        if self._engine is None:
            raise RPUBackendError(f"call .to('rpu') before {what}.")

    # ------------------------------------------------------------------ pre-processing
    def _get_processor(self):
        if self._processor is None:
            from transformers import AutoProcessor
            self._processor = AutoProcessor.from_pretrained(self._ckpt_dir, local_files_only=True)
        return self._processor

    def _build_raw_observation(self, *, images, instruction, proprioception, noise, noise_seed) -> dict:
        eng = self._engine
        cfg = eng.cfg
        if len(images) != self._n_cameras and self._n_cameras:
            raise ValueError(f"expected {self._n_cameras} camera images, got {len(images)}")
        proc = self._get_processor()
        enc = proc.image_processor(images=list(images), return_tensors="pt")
        tok = proc.tokenizer(instruction, truncation=True, max_length=self._max_lang_tokens, return_tensors="pt")
        state = torch.zeros(cfg.state_dim)
        if proprioception is not None:
            p = torch.as_tensor(proprioception, dtype=torch.float32).flatten()
            if p.numel() > cfg.state_dim:
                raise ValueError(f"proprioception has {p.numel()} values, the model takes at most {cfg.state_dim}")
            state[:p.numel()] = p
        if noise is None:
            noise = torch.randn(cfg.horizon, cfg.action_dim, generator=torch.Generator().manual_seed(int(noise_seed)))
        return {"pixel_values": enc["pixel_values"], "image_grid_thw": enc["image_grid_thw"],
                "lang_tokens": tok["input_ids"][0][tok["attention_mask"][0].bool()], "state": state, "noise": noise}

    def _run(self, obs: Mapping) -> torch.Tensor:
        eng = self._engine
        grid = torch.as_tensor(obs["image_grid_thw"])
        merge2 = eng.vlm.vcfg.spatial_merge_size ** 2
        per_image = [int(t * h * w) // merge2 for t, h, w in grid.tolist()]
        ids = eng.build_input_ids(per_image, torch.as_tensor(obs["lang_tokens"]))
        return eng.predict(ids, obs["pixel_values"], grid, torch.as_tensor(obs["state"], dtype=torch.float32),
                           torch.as_tensor(obs["noise"], dtype=torch.float32), use_graph=self._one_graph)

    # ------------------------------------------------------------------ graphs
    @_serialized
    def prepare_graphs(self, *, images=None, instruction=None, proprioception=None, noise=None, noise_seed: int = 0,
                       obs: Optional[Mapping] = None) -> "Lingbot2Policy":
        """BUILD the denoise graph on a representative observation, REPLAY it once, check that the replay reproduces
        the build bit for bit, and freeze: afterwards ``graphs_ready`` is True and ``graph_profile`` describes the
        prepared envelope."""
        self._require_ready("prepare_graphs()")
        if self._graph_profile is not None:
            raise RuntimeError("Lingbot2Policy graphs are already prepared")
        if obs is None:
            if images is None or instruction is None:
                raise ValueError("pass either obs=..., or images=... and instruction=...")
            obs = self._build_raw_observation(images=images, instruction=instruction, proprioception=proprioception,
                                              noise=noise, noise_seed=noise_seed)
        t0 = time.perf_counter()
        first = self._run(obs).float().cpu().clone()
        second = self._run(obs).float().cpu().clone()
        self._engine.check_status()
        if not torch.equal(first, second):
            raise RPUBackendError("LingBot-VLA-V2 graph replay did not reproduce the build run; graphs not frozen")
        self._prepare_ms["graph_warmup_ms"] = (time.perf_counter() - t0) * 1000.0
        self._graph_profile = {"num_steps": self._engine.cfg.num_steps, "max_prefix": self._engine.max_prefix,
                               "max_lang_tokens": self._max_lang_tokens, "graphs": len(self._engine._graphs),
                               "deterministic": True}
        return self

    # ------------------------------------------------------------------ inference
    @_serialized
    def infer(self, *, images=None, instruction=None, proprioception=None, noise=None, noise_seed: int = 0,
              obs: Optional[Mapping] = None) -> Lingbot2ActionOutput:
        self._require_ready("infer()")
        if obs is None:
            if images is None or instruction is None:
                raise ValueError("pass either obs=..., or images=... and instruction=...")
            obs = self._build_raw_observation(images=images, instruction=instruction, proprioception=proprioception,
                                              noise=noise, noise_seed=noise_seed)
        t0 = time.perf_counter()
        with torch.no_grad():
            raw = self._run(obs)
            full = raw.detach().float().cpu()              # the device->host copy ends the timed region
        latency_ms = (time.perf_counter() - t0) * 1000.0
        self._engine.check_status()
        if not bool(torch.isfinite(full).all()):
            raise RPUBackendError("LingBot-VLA-V2 produced a non-finite action chunk.")
        valid = min(VALID_ACTION_DIMS, full.shape[1])
        norm = full[:, :valid].contiguous()
        physical = None
        if self._denorm is not None:
            physical = self._denorm.unapply(norm, state=obs.get("state") if isinstance(obs, Mapping) else None).contiguous()
            if not bool(torch.isfinite(physical).all()):
                raise RPUBackendError("LingBot-VLA-V2 de-normalization produced a non-finite physical action chunk; "
                                      "refusing physical-unit output.")
        return Lingbot2ActionOutput(actions_normalized=norm, actions_full=full, latency_ms=latency_ms,
                                    phase_ms=dict(self._prepare_ms), actions_physical=physical,
                                    extra={"dtype": self._dtype, "valid_action_dims": valid,
                                           "denormalized": physical is not None, "robot_ready": physical is not None,
                                           "graphs_ready": self.graphs_ready})

    def predict_action_chunk(self, **kwargs: Any) -> torch.Tensor:
        """Just the ``[H, 16]`` real-DoF action chunk in physical units."""
        return self.infer(**kwargs).actions

    def close(self) -> None:
        with self._lock:
            if self._closed:
                return
            self._closed = True
            eng, self._engine = self._engine, None
            if eng is not None:
                eng.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


__all__ = ["Lingbot2Policy", "Lingbot2ActionOutput", "VALID_ACTION_DIMS"]
