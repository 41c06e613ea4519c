"""``WallOssPolicy``: public facade of the Wall-OSS policy (Qwen2.5-VL prompt decoder + flow-matching action decoder).

    policy = WallOssPolicy.from_checkpoint(ckpt_dir, dataset_key="berkeley_autolab_ur5", camera_names=("face_view",)).to("rpu")
    policy.prepare_graphs(images=[...], instruction="...", proprioception=[...])   # optional: BUILD + check + freeze
    out = policy.infer(images=[...], instruction="...", proprioception=[...])      # WallOssActionOutput
    out.actions      # [horizon, action_dim] physical units (de-normalised with the checkpoint's per-dataset statistics)
    out.latency_ms
    policy.close()

The checkpoint, the camera roster, the dataset key (normaliser entry and embodiment tag of the prompt) and the precision
are fixed at construction; pixels, instruction, proprioception, noise and the degree-of-freedom mask change per call.
``obs=`` accepts an already pre-processed observation (``input_ids``, ``pixel_values``, ``image_grid_thw``, ``noise``,
optionally ``dof_mask``), which also lets the policy run without the processor files.

The real-time-chunking profile of the reference (``rtc=True``: committed action prefix, per-token flow time) is an
evaluation-only path there and is not built here; asking for it raises ``UnsupportedModelError``.

Reference: ``python/rpu_backend/api/wall_oss.py:230-241,303-345,638-775,803-1046``.
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
from .errors import RPUBackendError, UnsupportedModelError

_RUNTIME_ENV_ALLOWLIST = frozenset({"RPU_WALL_OSS_FUSED_DENOISE", "RPU_WARMUP"})
_QUANT_FLAGS = ("w8a16", "w4a16", "nvfp4a16")


@dataclasses.dataclass(frozen=True)
class WallOssActionOutput:
    actions: torch.Tensor            # [horizon, action_dim] physical units, CPU fp32
    action_hz: float
    latency_ms: float
    phase_ms: Dict[str, float]
    extra: Dict[str, Any] = dataclasses.field(default_factory=dict)


def _int_at_least(name: str, value, minimum: int) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < minimum:
        raise ValueError(f"{name} must be an integer >= {minimum}, got {value!r}")
    return value


def _cpu_finite(value, *, name: str) -> torch.Tensor:
    t = torch.as_tensor(value).detach().to("cpu", torch.float32)
    if not bool(torch.isfinite(t).all()):
        raise ValueError(f"{name} must contain only finite values")
    return t


def _binary(value, *, name: str) -> torch.Tensor:
    t = _cpu_finite(value, name=name)
    if not bool(((t == 0) | (t == 1)).all()):
        raise ValueError(f"{name} must contain only 0 or 1")
    return t


def _serialized(method):
    """One call into the policy at a time: the engine's graph inputs are shared static buffers."""
    def wrapped(self, *args, **kwargs):
        with self._lock:
            return method(self, *args, **kwargs)
    wrapped.__name__, wrapped.__doc__ = method.__name__, method.__doc__
    return wrapped


class WallOssPolicy:
    FAMILY = "Wall-OSS (Qwen2.5-VL backbone with a flow-matching action expert)"

    def __init__(self) -> None:
        raise RuntimeError("WallOssPolicy() is not a public constructor. Use WallOssPolicy.from_checkpoint(...).to('rpu').")

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_checkpoint(cls, ckpt_dir, *, dataset_key: str = "berkeley_autolab_ur5", camera_names: Sequence[str] = ("face_view",),
                        delta_action: bool = False, state_bins: int = 256, action_hz: float = 32.0, action_horizon: int = 32,
                        num_steps: int = 10, max_seq_len: int = 2048, dtype: str = "fp16", w8a16: bool = False,
                        w4a16: bool = False, nvfp4a16: bool = False, fp16_ckpt_dir=None,
                        active_slots: Optional[Sequence[int]] = None, runtime_env: Optional[Mapping] = None,
                        rpu_execution=None, rtc: bool = False, prompt_style: str = "default",
                        causal_action_attention_mask: bool = True) -> "WallOssPolicy":
        """Bind a policy to a checkpoint directory (``config.json``, safetensors shards, the Qwen2.5-VL processor files,
        ``normalizer_action.pth`` / ``normalizer_propri.pth``).  Nothing is read yet; ``.to('rpu')`` builds the runtime.
        Argument errors are raised here, before any weight is touched."""
        from ..adapters.wall_oss import CAMERA_PROSE, PROMPT_STYLES
        from ._execution import normalize_rpu_execution
        for flag, on in zip(_QUANT_FLAGS, (w8a16, w4a16, nvfp4a16)):
            if not isinstance(on, bool):
                raise TypeError(f"{flag} must be bool, got {on!r}")
        if sum((w8a16, w4a16, nvfp4a16)) > 1:
            raise ValueError("Wall-OSS precision modes are mutually exclusive")
        if w8a16 or w4a16 or nvfp4a16:
            raise UnsupportedModelError("Wall-OSS runs in 16 bits (fp16 / bf16) in this framework; the quantised checkpoints "
                                        "made by rpu_backend.quant.convert_wall_oss* are not loaded by this policy")
        if not isinstance(rtc, bool):
            raise TypeError(f"rtc must be bool, got {rtc!r}")
        if rtc:
            raise UnsupportedModelError("the Wall-OSS real-time-chunking profile (rtc=True) is not built in this framework")
        if dtype not in ("fp16", "bf16"):
            raise ValueError(f"dtype must be fp16 or bf16, got {dtype!r}")
        if not isinstance(dataset_key, str) or not dataset_key:
            raise ValueError("dataset_key must be a non-empty string")
        cams = list(camera_names)
        if not cams or any(c not in CAMERA_PROSE for c in cams):
            raise ValueError(f"camera_names must be a non-empty list out of {sorted(CAMERA_PROSE)}, got {cams!r}")
        if prompt_style not in PROMPT_STYLES:
            raise ValueError(f"prompt_style must be one of {PROMPT_STYLES}, got {prompt_style!r}")
        if isinstance(action_hz, bool) or not isinstance(action_hz, (int, float)) or not action_hz > 0:
            raise ValueError(f"action_hz must be a positive number, got {action_hz!r}")
        slots = None
        if active_slots is not None:
            slots = [_int_at_least("active_slots entry", s, 0) for s in active_slots]
            if not slots or len(set(slots)) != len(slots):
                raise ValueError("active_slots must be a non-empty list of distinct indices")
        self = object.__new__(cls)
        self._ckpt_dir = os.fspath(ckpt_dir)
        self._dataset_key, self._camera_names, self._delta_action = dataset_key, cams, bool(delta_action)
        self._state_bins = _int_at_least("state_bins", state_bins, 2)
        self._action_hz = float(action_hz)
        self._action_horizon = _int_at_least("action_horizon", action_horizon, 1)
        self._num_steps = _int_at_least("num_steps", num_steps, 1)
        self._max_seq_len = _int_at_least("max_seq_len", max_seq_len, self._action_horizon + 16)
        self._dtype, self._prompt_style, self._causal = dtype, prompt_style, bool(causal_action_attention_mask)
        self._active_slots = slots
        self._execution = normalize_rpu_execution(rpu_execution, entry_point="WallOssPolicy.from_checkpoint",
                                                  supported={"prefill": ("chunk_size", "padding_rows", "padding_budget"),
                                                             "vision": ("chunk_size",), "action": ("chunk_size",)})
        self._runtime_env = normalize_runtime_env(runtime_env, owner="WallOssPolicy", allowed=_RUNTIME_ENV_ALLOWLIST)
        self._init_state()
        return self

    from_pretrained = from_checkpoint

    def _init_state(self) -> None:
        self._engine = self._processor = self._normalizer = None
        self._closed, self._one_graph = False, True
        self._lock = threading.RLock()
        self._prepare_ms: Dict[str, float] = {}
        self._graph_profile: Optional[dict] = None

    @classmethod
    def _from_engine(cls, engine, *, normalizer=None, action_hz: float = 32.0, active_slots=None) -> "WallOssPolicy":
        """A policy over an already built engine (tests, applications that assemble the runtime themselves)."""
        self = object.__new__(cls)
        self._ckpt_dir, self._dataset_key = None, getattr(normalizer, "dataset_key", "")
        self._camera_names, self._delta_action, self._state_bins = [], False, 256
        self._action_hz, self._action_horizon, self._num_steps = float(action_hz), engine.cfg.horizon, engine.cfg.num_steps
        self._max_seq_len = engine.max_seq
        self._dtype = "fp16" if engine.dtype == torch.float16 else "bf16"
        self._prompt_style, self._causal, self._active_slots = "default", engine.cfg.causal_actions, active_slots
        self._execution, self._runtime_env = {}, {}
        self._init_state()
        self._engine, self._normalizer = engine, normalizer
        return self

    # ------------------------------------------------------------------ properties
    @property
    def action_dim(self) -> int:
        self._require_ready("action_dim")
        return self._engine.cfg.action_dim

    @property
    def action_horizon(self) -> int:
        return self._action_horizon

    @property
    def camera_names(self) -> list:
        return list(self._camera_names)

    @property
    def precision(self) -> str:
        return self._dtype

    @property
    def graphs_ready(self) -> bool:
        return self._engine is not None and not self._closed and self._graph_profile is not None

    @property
    def graph_profile(self) -> Optional[dict]:
        return None if not self.graphs_ready else dict(self._graph_profile)

    # ------------------------------------------------------------------ build
    @_serialized
    def to(self, device: Any) -> "WallOssPolicy":
        from ..runtime.device import resolve_device
        if self._closed:
            raise RPUBackendError("WallOssPolicy is closed")
        dev = resolve_device(device)
        if dev.type != "cuda":
            raise RPUBackendError(f"WallOssPolicy runs on the accelerator only, got device {device!r}")
        if self._engine is not None:
            return self
        from ..adapters.wall_oss import Normalizer, build_engine
        from ..runtime.control import rpu_env_bool
        from ._loading import checkpoint_tensor_getter
        self._normalizer = Normalizer.from_dir(self._ckpt_dir, self._dataset_key)   # configuration errors before weights
        t0 = time.perf_counter()
        with open(os.path.join(self._ckpt_dir, "config.json"), "r", encoding="utf-8") as f:
            config = json.load(f)
        get = checkpoint_tensor_getter(self._ckpt_dir)
        old_env = {k: os.environ.get(k) for k in self._runtime_env}
        os.environ.update(self._runtime_env)
        try:
            self._one_graph = rpu_env_bool("RPU_WALL_OSS_FUSED_DENOISE", True)      # 0: one launch sequence per Euler step
            self._engine = build_engine(config, get, horizon=self._action_horizon, num_steps=self._num_steps,
                                        max_seq_len=self._max_seq_len, causal_actions=self._causal, device=dev,
                                        dtype=torch.float16 if self._dtype == "fp16" else torch.bfloat16)
        finally:
            for k, v in old_env.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
        self._prepare_ms["build_ms"] = (time.perf_counter() - t0) * 1000.0
        return self

    def _require_ready(self, what: str) -> None:
        if self._closed:
            raise RPUBackendError("WallOssPolicy is closed")
        if self._engine is None:
            raise RPUBackendError(f"WallOssPolicy.to('rpu') must own a complete live runtime before {what}.")

    # ------------------------------------------------------------------ inputs
    def _get_processor(self):
        if self._processor is None:
            from transformers import AutoProcessor
            self._processor = AutoProcessor.from_pretrained(self._ckpt_dir, local_files_only=True)
        return self._processor

    def _default_dof_mask(self) -> torch.Tensor:
        H, AD = self._action_horizon, self._engine.cfg.action_dim
        if self._active_slots is None:
            return torch.ones(H, AD)
        row = torch.zeros(AD)
        for s in self._active_slots:
            if s >= AD:
                raise ValueError(f"active_slots entry {s} exceeds action_dim={AD}")
            row[s] = 1.0
        return row[None].expand(H, AD).clone()

    def _grid(self, value, *, name: str, binary: bool = False) -> torch.Tensor:
        H, AD = self._action_horizon, self._engine.cfg.action_dim
        t = _binary(value, name=name) if binary else _cpu_finite(value, name=name)
        if tuple(t.shape) == (1, H, AD):
            t = t[0]
        if tuple(t.shape) != (H, AD):
            raise ValueError(f"{name} shape {tuple(t.shape)} != expected {(H, AD)}")
        return t.contiguous()

    def _build_observation(self, *, images, instruction, proprioception, state_mask) -> dict:
        from ..adapters.wall_oss import build_flow_prompt, expand_image_tokens
        image_list = list(images) if isinstance(images, (list, tuple)) else [images]
        if len(image_list) != len(self._camera_names):
            raise ValueError(f"WallOssPolicy expected {len(self._camera_names)} images for camera_names={self._camera_names}, "
                             f"got {len(image_list)}")
        if any(im is None for im in image_list):
            raise ValueError("WallOssPolicy images must not contain None")
        if not isinstance(instruction, str) or not instruction.strip():
            raise ValueError("WallOssPolicy instruction must be a non-empty string")
        prop = _cpu_finite(proprioception, name="proprioception").reshape(-1)
        mask = torch.ones_like(prop) if state_mask is None else _binary(state_mask, name="state_mask").reshape(-1)
        if mask.numel() != prop.numel():
            raise ValueError(f"WallOssPolicy state_mask has {mask.numel()} entries but proprioception has {prop.numel()}")
        state = self._normalizer.state_string(prop, mask, self._state_bins)
        text = build_flow_prompt(instruction, self._camera_names, self._dataset_key, self._delta_action, state,
                                 style=self._prompt_style)
        proc = self._get_processor()
        enc = proc.image_processor(images=image_list, return_tensors="pt")
        grid = enc["image_grid_thw"]
        text = expand_image_tokens(text, grid, proc.image_processor.merge_size)
        ids = proc.tokenizer([text], return_tensors="pt")["input_ids"][0]
        return {"input_ids": ids, "pixel_values": enc["pixel_values"].float(), "image_grid_thw": grid, "text": text}

    def _complete(self, obs: Mapping, noise, dof_mask, noise_seed: int) -> dict:
        H, AD = self._action_horizon, self._engine.cfg.action_dim
        obs = dict(obs)
        if noise is None and obs.get("noise") is None:
            obs["noise"] = torch.randn((H, AD), generator=torch.Generator().manual_seed(int(noise_seed)))
        else:
            obs["noise"] = self._grid(noise if noise is not None else obs["noise"], name="noise")
        dm = dof_mask if dof_mask is not None else obs.get("dof_mask")
        obs["dof_mask"] = self._default_dof_mask() if dm is None else self._grid(dm, name="dof_mask", binary=True)
        return obs

    def _run(self, obs: Mapping, num_steps: int) -> torch.Tensor:
        eng = self._engine
        pad = None
        if not bool((obs["dof_mask"] == 1).all()):
            if self._normalizer is None:
                raise RPUBackendError("a dof_mask with inactive dimensions needs the action normalizer (normalised physical zero)")
            pad = self._normalizer.padding_action(self._action_horizon)
        return eng.predict(torch.as_tensor(obs["input_ids"]), obs.get("pixel_values"), obs.get("image_grid_thw"), obs["noise"],
                           obs["dof_mask"], num_steps, padding_action=pad, use_graph=self._one_graph)

    # ------------------------------------------------------------------ graphs
    @_serialized
    def prepare_graphs(self, *, images=None, instruction=None, proprioception=None, state_mask=None, noise=None,
                       dof_mask=None, num_steps: Optional[int] = None, noise_seed: int = 0,
                       obs: Optional[Mapping] = None) -> "WallOssPolicy":
        """BUILD the denoise graph on a representative observation, REPLAY it once, check that the replay reproduces
        the build bit for bit, and freeze: afterwards ``graphs_ready`` is True and ``graph_profile`` describes the
        prepared envelope (an ``infer`` with another ``num_steps`` or mask kind is then refused, not built online)."""
        self._require_ready("prepare_graphs()")
        if self._graph_profile is not None:
            raise RuntimeError("WallOssPolicy graphs are already prepared")
        steps = self._num_steps if num_steps is None else _int_at_least("num_steps", num_steps, 1)
        if obs is None:
            if images is None or instruction is None or proprioception is None:
                raise ValueError("pass either obs=..., or images=..., instruction=... and proprioception=...")
            obs = self._build_observation(images=images, instruction=instruction, proprioception=proprioception,
                                          state_mask=state_mask)
        obs = self._complete(obs, noise, dof_mask, noise_seed)
        t0 = time.perf_counter()
        first = self._run(obs, steps).float().cpu().clone()
        second = self._run(obs, steps).float().cpu().clone()
        self._engine.check_status()
        if not torch.equal(first, second):
            raise RPUBackendError("Wall-OSS graph replay did not reproduce the build run; graphs not frozen")
        self._prepare_ms["graph_warmup_ms"] = (time.perf_counter() - t0) * 1000.0
        self._graph_profile = {"num_steps": steps, "horizon": self._action_horizon, "max_prefix": self._engine.max_prefix,
                               "masked_dof": not bool((obs["dof_mask"] == 1).all()), "graphs": len(self._engine._graphs),
                               "deterministic": True}
        return self

    # ------------------------------------------------------------------ inference
    @_serialized
    def infer(self, *, images=None, instruction=None, proprioception=None, state_mask=None, noise=None, dof_mask=None,
              num_steps: Optional[int] = None, noise_seed: int = 0, rtc_prefix_actions=None, inference_delay: int = 0,
              use_rtc: bool = False, obs: Optional[Mapping] = None) -> WallOssActionOutput:
        """One action chunk: CPU fp32 physical-unit actions ``[horizon, action_dim]`` and the wall time of the call
        (pre-processing, prompt prefill, denoise loop, device-to-host copy, de-normalisation)."""
        self._require_ready("inference")
        if use_rtc or inference_delay or rtc_prefix_actions is not None:
            raise UnsupportedModelError("this WallOssPolicy was not built with rtc=True (real-time chunking is not built)")
        steps = self._num_steps if num_steps is None else _int_at_least("num_steps", num_steps, 1)
        _int_at_least("noise_seed", noise_seed, 0)
        t0 = time.perf_counter()
        if obs is None:
            if images is None or instruction is None or proprioception is None:
                raise ValueError("pass either obs=..., or images=..., instruction=... and proprioception=...")
            obs = self._build_observation(images=images, instruction=instruction, proprioception=proprioception,
                                          state_mask=state_mask)
        obs = self._complete(obs, noise, dof_mask, noise_seed)
        masked = not bool((obs["dof_mask"] == 1).all())
        if self._graph_profile is not None and (steps != self._graph_profile["num_steps"] or masked != self._graph_profile["masked_dof"]):
            raise RPUBackendError("request is outside the prepared graph profile "
                                  f"(num_steps={steps}, masked_dof={masked}); online graph BUILD is disabled")
        t1 = time.perf_counter()
        with torch.no_grad():
            x = self._run(obs, steps).detach().float().cpu()          # the device->host copy ends the device phase
        t2 = time.perf_counter()
        self._engine.check_status()
        if not bool(torch.isfinite(x).all()):
            raise RPUBackendError("WallOssPolicy runtime action contains non-finite values")
        actions = x if self._normalizer is None else self._normalizer.denormalize(x)
        actions = actions.contiguous()
        t3 = time.perf_counter()
        return WallOssActionOutput(
            actions=actions, action_hz=self._action_hz, latency_ms=(t3 - t0) * 1000.0,
            phase_ms={"preprocess_ms": (t1 - t0) * 1000.0, "device_ms": (t2 - t1) * 1000.0, "postprocess_ms": (t3 - t2) * 1000.0},
            extra={"ckpt_dir": self._ckpt_dir, "dataset_key": self._dataset_key, "prefix_len": int(torch.as_tensor(obs["input_ids"]).numel()),
                   "real_prefix_len": int(torch.as_tensor(obs["input_ids"]).numel()), "num_images": len(self._camera_names),
                   "num_steps": steps, "action_chunk_size_resolved": (self._action_horizon + 15) // 16 * 16, "use_rtc": False,
                   "inference_delay": 0, "noise_seed": int(noise_seed), "prepare_ms": dict(self._prepare_ms),
                   "graphs_ready": self.graphs_ready, "precision": self.precision, "x_norm": x,
                   "denormalized": self._normalizer is not None})

    def predict_action_chunk(self, **kwargs: Any) -> torch.Tensor:
        """Just the CPU physical action chunk ``[horizon, action_dim]``."""
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


__all__ = ["WallOssPolicy", "WallOssActionOutput"]
