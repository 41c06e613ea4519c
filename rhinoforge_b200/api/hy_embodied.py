"""``HyEmbodiedPolicy``: public facade of the Hy-Embodied VLA (HYViT2 tower, HunYuan-VL mixture-of-transformers prefill,
flow-matching action expert).

    policy = HyEmbodiedPolicy.from_checkpoint(ckpt_dir, norm_stats_path=".../norm_stats.json").to("rpu")
    out = policy.infer(images=[cam0, cam1, cam2], instruction="...", ee_pose=current_dual_arm_pose_wxyz)
    out.actions             # [H - 1, 16] physical dual-arm poses (needs the statistics and ee_pose)
    out.actions_normalized  # [50, 20] normalised relative increments;  out.actions_full: [50, 32];  out.latency_ms
    policy.close()

The model emits NORMALISED relative pose increments; physical poses need the checkpoint's normalisation statistics and
the current end-effector pose.  The statistics are read from a JSON file or passed as a mapping; a pickle file is only
opened when the caller explicitly trusts it AND gives its exact SHA-256.  ``obs=`` accepts an already pre-processed
observation (``adapters.hy_vla.build_observation``), which also lets the policy run without tokenizer files.

Reference: ``python/rpu_backend/api/hy_embodied.py:294-340,343-520,719-876``.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import threading
import time
from collections.abc import Mapping, Sequence
from typing import Any, Dict, Optional

import torch

from ._runtime_env import normalize_runtime_env
from .errors import RPUBackendError, RPUConfigError, UnsupportedModelError

VALID_ACTION_DIMS = 20
_RUNTIME_ENV_ALLOWLIST = frozenset({"RPU_HY_VLA_UNROLL", "RPU_WARMUP"})
_DTYPES = ("fp16", "bf16")
_OBS_KEYS = ("images", "lang_tokens", "prefill_mask", "prefill_pos", "modality_mask", "denoise_mask", "suffix_pos", "noise",
             "state", "n_valid")


@dataclasses.dataclass(frozen=True)
class HyEmbodiedActionOutput:
    """One action chunk.  ``actions`` raises unless this call decoded physical poses: a normalised increment must never be
    sent to a robot as a pose by accident."""

    actions_normalized: torch.Tensor       # [n_action, 20]
    actions_full: torch.Tensor             # [n_action, action_dim]
    latency_ms: float
    phase_ms: Dict[str, float]
    actions_physical: Any = None           # numpy [H - 1, 16] (wxyz), None without statistics + ee_pose
    extra: Dict[str, Any] = dataclasses.field(default_factory=dict)

    @property
    def actions(self):
        if self.actions_physical is None:
            raise RPUBackendError(
                "Hy-Embodied actions are normalized relative increments, not poses: build the policy with "
                "norm_stats_path=... and call infer(..., ee_pose=<current dual-arm pose, 16 values, wxyz>) to get physical "
                "poses; read .actions_normalized / .actions_full to inspect the normalized grid on purpose.")
        return self.actions_physical

    @property
    def physical_action_available(self) -> bool:
        """True iff THIS call produced physical poses (statistics configured and ``ee_pose`` given).  It says the output
        has physical units, not that those units and frames match a particular robot."""
        return self.actions_physical is not None


def _load_norm_stats(path: str, *, trust_pickle: bool, sha256: Optional[str]) -> Mapping:
    if path.endswith(".json"):
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    # any other extension is treated as a pickle: executable on load, so both an explicit opt-in and the exact digest
    if not trust_pickle or not sha256:
        raise RPUConfigError(f"{path!r} is not JSON; a pickle is only read with trust_norm_stats_pickle=True and "
                             "norm_stats_sha256=<its exact SHA-256> (convert it to JSON to avoid executing it)")
    with open(path, "rb") as f:
        blob = f.read()
    digest = hashlib.sha256(blob).hexdigest()
    if digest != sha256.strip().lower():
        raise RPUConfigError(f"{path!r} has SHA-256 {digest}, not the trusted {sha256!r}; refusing to unpickle")
    import pickle
    return pickle.loads(blob)


def _serialized(method):
    def wrapped(self, *args, **kwargs):
        with self._lock:
            return method(self, *args, **kwargs)
    wrapped.__name__, wrapped.__doc__ = method.__name__, method.__doc__
    return wrapped


class HyEmbodiedPolicy:
    FAMILY = "HunYuan embodied VLA (HYViT2 tower, twin-weight prefill, action expert)"

    def __init__(self) -> None:
        raise RuntimeError("HyEmbodiedPolicy() is not a public constructor. Use HyEmbodiedPolicy.from_checkpoint(...).to('rpu').")

    @classmethod
    def from_checkpoint(cls, ckpt_dir, *, dtype: str = "fp16", prefix_len: int = 240, n_cameras: int = 3, norm_stats_path=None,
                        norm_stats: Optional[Mapping] = None, trust_norm_stats_pickle: bool = False,
                        norm_stats_sha256: Optional[str] = None, umi_coord_frame: bool = True, umi_gripper_space: bool = False,
                        runtime_env: Optional[Mapping] = None, threads: int = 12) -> "HyEmbodiedPolicy":
        """Bind a policy to a checkpoint directory (``model.safetensors`` and, for raw observations, the tokenizer
        files).  Argument errors are raised here, before any weight is read."""
        dtype = (dtype or "fp16").strip().lower()
        if dtype not in _DTYPES:
            if dtype.startswith(("w8a16", "w4a16")):
                raise UnsupportedModelError(f"Hy-Embodied precision profile {dtype!r} is not built in this framework (fp16 / bf16)")
            raise ValueError(f"dtype must be one of {_DTYPES}, got {dtype!r}")
        if isinstance(prefix_len, bool) or not isinstance(prefix_len, int) or prefix_len % 16 or not 16 <= prefix_len <= 240:
            raise ValueError(f"prefix_len must be a multiple of 16 in [16, 240], got {prefix_len!r}")
        if isinstance(n_cameras, bool) or not isinstance(n_cameras, int) or n_cameras <= 0:
            raise ValueError(f"n_cameras must be a positive integer, got {n_cameras!r}")
        if not isinstance(trust_norm_stats_pickle, bool):
            raise TypeError("trust_norm_stats_pickle must be bool")
        if norm_stats is not None and norm_stats_path is not None:
            raise ValueError("give norm_stats (a mapping) or norm_stats_path, not both")
        self = object.__new__(cls)
        self._ckpt_dir, self._dtype, self._prefix_len, self._n_cameras = os.fspath(ckpt_dir), dtype, prefix_len, n_cameras
        self._norm_stats_path = None if norm_stats_path is None else os.fspath(norm_stats_path)
        self._norm_stats, self._trust, self._sha = norm_stats, trust_norm_stats_pickle, norm_stats_sha256
        self._umi_frame, self._umi_gripper = bool(umi_coord_frame), bool(umi_gripper_space)
        self._runtime_env = normalize_runtime_env(runtime_env, owner="HyEmbodiedPolicy", allowed=_RUNTIME_ENV_ALLOWLIST)
        self._threads = int(threads)
        self._init_state()
        return self

    from_pretrained = from_checkpoint

    def _init_state(self) -> None:
        self._engine = self._decoder = self._tok = None
        self._closed, self._one_graph = False, True
        self._lock = threading.RLock()
        self._prepare_ms: Dict[str, float] = {}

    @classmethod
    def _from_engine(cls, engine, *, decoder=None, prefix_len: int = 240, n_cameras: int = 3) -> "HyEmbodiedPolicy":
        """A policy over an already built engine (tests, applications that assemble the runtime themselves)."""
        self = object.__new__(cls)
        self._ckpt_dir, self._dtype = None, "fp16" if engine.dtype == torch.float16 else "bf16"
        self._prefix_len, self._n_cameras = prefix_len, n_cameras
        self._norm_stats_path = self._norm_stats = self._sha = None
        self._trust, self._umi_frame, self._umi_gripper, self._runtime_env, self._threads = False, True, False, {}, 12
        self._init_state()
        self._engine, self._decoder = engine, decoder
        return self

    # ------------------------------------------------------------------ properties
    dtype = property(lambda self: self._dtype)
    prefix_len = property(lambda self: self._prefix_len)
    action_decode_configured = property(lambda self: self._decoder is not None)

    @property
    def action_dim(self) -> int:
        return VALID_ACTION_DIMS

    @property
    def model_horizon(self) -> int:
        self._require_ready("model_horizon")
        return self._engine.cfg.n_action

    @property
    def camera_names(self) -> list:
        from ..adapters.hy_vla import CAMERA_ORDER
        return list(CAMERA_ORDER)[:self._n_cameras]

    # ------------------------------------------------------------------ build
    def _build_decoder(self):
        from .hy_action_decode import HyVlaActionDecoder
        info = self._norm_stats
        if info is None and self._norm_stats_path is not None:
            info = _load_norm_stats(self._norm_stats_path, trust_pickle=self._trust, sha256=self._sha)
        if info is None:
            return None
        return HyVlaActionDecoder.from_norm_stats_mapping(info, umi_coord_frame=self._umi_frame, umi_gripper_space=self._umi_gripper)

    @_serialized
    def to(self, device: Any) -> "HyEmbodiedPolicy":
        from ..runtime.device import resolve_device
        if self._closed:
            raise RPUBackendError("HyEmbodiedPolicy is closed")
        dev = resolve_device(device)
        if dev.type != "cuda":
            raise RPUBackendError(f"HyEmbodiedPolicy runs on the accelerator only, got device {device!r}")
        if self._engine is not None:
            return self
        self._decoder = self._build_decoder()                     # configuration errors first, before weights are read
        from ..adapters.hy_vla.runtime import build_engine
        from ..runtime.control import rpu_env_bool
        from ._loading import checkpoint_tensor_getter
        t0 = time.perf_counter()
        get = checkpoint_tensor_getter(self._ckpt_dir)
        old_env = {k: os.environ.get(k) for k in self._runtime_env}
        os.environ.update(self._runtime_env)
        try:
            self._one_graph = rpu_env_bool("RPU_HY_VLA_UNROLL", True)      # 0: one launch sequence per Euler step
            self._engine = build_engine(get, names=get.names, prefix_len=self._prefix_len, n_cameras=self._n_cameras, device=dev,
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
            raise RPUBackendError("HyEmbodiedPolicy is closed")
        if self._engine is None:
            raise RPUBackendError(f"call .to('rpu') before {what}.")

    def _tokenizer(self):
        if self._tok is None:
            from transformers import AutoTokenizer
            self._tok = AutoTokenizer.from_pretrained(self._ckpt_dir, local_files_only=True)
        return self._tok

    # ------------------------------------------------------------------ inference
    @_serialized
    def infer(self, *, images: Optional[Sequence[Any]] = None, instruction: Optional[str] = None, ee_pose: Any = None,
              state: Any = None, noise: Optional[torch.Tensor] = None, noise_seed: Optional[int] = None,
              obs: Optional[Mapping[str, Any]] = None) -> HyEmbodiedActionOutput:
        """One action chunk.  Either a raw observation (``images`` + ``instruction``, with ``ee_pose`` or a normalised
        ``state``) that the policy pre-processes itself, or ``obs=`` with a ready observation; the two do not mix."""
        self._require_ready("infer()")
        if ee_pose is not None and state is not None:
            raise ValueError("give ee_pose (a raw pose) or state (already normalized), not both")
        if obs is not None:
            if any(v is not None for v in (images, instruction, ee_pose, state, noise, noise_seed)):
                raise ValueError("obs= does not mix with images / instruction / ee_pose / state / noise: the run would silently "
                                 "use one and ignore the other")
            missing = [k for k in _OBS_KEYS if k not in obs]
            if missing:
                raise ValueError(f"obs lacks {missing}")
        else:
            if images is None or instruction is None:
                raise ValueError("pass either obs=..., or images=... and instruction=...")
            if len(images) != self._n_cameras:
                raise ValueError(f"expected {self._n_cameras} camera images, got {len(images)}")
        from ..adapters.hy_vla import build_observation
        from ..adapters.hy_vla.runtime import get_action
        eng = self._engine
        cfg = eng.cfg
        t0 = time.perf_counter()
        if obs is None:
            if ee_pose is not None:
                if self._decoder is None:
                    raise RPUBackendError("ee_pose needs the normalization statistics (norm_stats_path=...) to be encoded")
                state = self._decoder.encode_state(ee_pose)
            obs = build_observation(images, instruction, self._tokenizer(), state=state, noise=noise, noise_seed=noise_seed,
                                    grid=cfg.grid, max_state_dim=cfg.state_dim, max_action_dim=cfg.action_dim,
                                    n_action=cfg.n_action)
        n_valid = obs["n_valid"]
        if isinstance(n_valid, bool) or not isinstance(n_valid, int) or n_valid <= 0:
            raise ValueError(f"obs['n_valid'] must be a positive integer, got {n_valid!r}")
        if (n_valid + 15) // 16 * 16 > self._prefix_len:
            raise RPUBackendError(f"the observation has {n_valid} real prefix rows; ceil16 exceeds prefix_len={self._prefix_len}: "
                                  "the prefix would be cut")
        t1 = time.perf_counter()
        with torch.no_grad():
            full = get_action(eng, obs, prefix_len=self._prefix_len, use_graph=self._one_graph).detach().float().cpu()
        t2 = time.perf_counter()
        eng.check_status()
        if not bool(torch.isfinite(full).all()):
            raise RPUBackendError("Hy-Embodied produced a non-finite action chunk.")
        norm = full[:, :min(VALID_ACTION_DIMS, full.shape[1])].contiguous()
        physical = None
        if self._decoder is not None and ee_pose is not None:
            physical = self._decoder.decode(norm.numpy(), ee_pose)
        t3 = time.perf_counter()
        return HyEmbodiedActionOutput(
            actions_normalized=norm, actions_full=full, latency_ms=(t3 - t0) * 1000.0,
            phase_ms={"preprocess_ms": (t1 - t0) * 1000.0, "device_ms": (t2 - t1) * 1000.0, "decode_ms": (t3 - t2) * 1000.0},
            actions_physical=physical,
            extra={"dtype": self._dtype, "prefix_len": self._prefix_len, "n_valid": int(n_valid), "prepare_ms": dict(self._prepare_ms),
                   "action_decode_configured": self.action_decode_configured})

    def predict_action_chunk(self, **kwargs: Any):
        """Just the physical dual-arm poses ``[H - 1, 16]``."""
        return self.infer(**kwargs).actions

    def close(self) -> None:
        with self._lock:
            if self._closed:
                return
            self._closed = True
            eng, self._engine = self._engine, None
            if eng is not None:
                tower = getattr(eng, "vision_tower", None)
                eng.close()
                if tower is not None:
                    tower.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


__all__ = ["HyEmbodiedPolicy", "HyEmbodiedActionOutput", "VALID_ACTION_DIMS"]
