"""``Pi05Policy``: public facade of the Pi0.5 vision-language-action policy.

    policy = Pi05Policy.from_pretrained(ckpt, rpu_execution=cfg, trust_remote_code=False).to("rpu")
    policy.prepare_graphs(batch, num_steps=10)                  # optional: BUILD + determinism check + freeze
    actions = policy.predict_action_chunk(batch, num_steps=10)  # [B, horizon, action_dim]
    a = policy.select_action(batch)                             # one step from the queued chunk

``batch`` follows the LeRobot convention: ``observation.images.<camera>`` ``[B,3,H,W]`` floats in
``[0,1]``, ``observation.language.tokens`` / ``observation.language.attention_mask`` ``[B,L]`` (the
tokenised prompt with the discretised state, as produced by the policy's pre-processor), optionally
``noise`` ``[B, horizon, action_dim]``.  Missing cameras are masked out, not zero-filled.
Reference: ``python/rpu_backend/api/policy.py:57-119,164-190,193-289``.
"""
from __future__ import annotations

import dataclasses
from collections import deque
from typing import Any, Dict, Optional

import torch

from ._execution import normalize_rpu_execution
from .errors import RPUBackendError, RPUUnsupportedDtypeError

IMAGE_PREFIX = "observation.images."
TOKENS_KEY = "observation.language.tokens"
TOKEN_MASK_KEY = "observation.language.attention_mask"
_STAGES = {"prefill": ("chunk_size", "padding_rows", "padding_budget"), "vision": ("chunk_size",), "action": ("chunk_size",)}


def _validate_batch(batch, *, entry_point: str) -> dict:
    if not isinstance(batch, dict):
        raise TypeError(f"{entry_point}: batch must be a dict, got {type(batch).__name__}")
    return batch


def _validate_num_steps(num_steps, *, entry_point: str):
    if num_steps is None:
        return None
    if isinstance(num_steps, bool) or not isinstance(num_steps, int) or num_steps < 1:
        raise ValueError(f"{entry_point}: num_steps must be a positive integer, got {num_steps!r}")
    return num_steps


def resize_with_pad(img: torch.Tensor, size: int) -> torch.Tensor:
    """``[B,3,H,W]`` in ``[0,1]`` -> ``[B,3,size,size]`` in ``[-1,1]``: aspect-preserving bilinear resize,
    centred, padded with -1 (black)."""
    B, C, H, W = img.shape
    if (H, W) != (size, size):
        r = max(W / size, H / size)
        nh, nw = int(H / r), int(W / r)
        img = torch.nn.functional.interpolate(img, size=(nh, nw), mode="bilinear", align_corners=False)
        ph, pw = size - nh, size - nw
        img = torch.nn.functional.pad(img, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2), value=0.0)
        mask = torch.zeros(1, 1, size, size, dtype=torch.bool, device=img.device)
        mask[..., ph // 2:ph // 2 + nh, pw // 2:pw // 2 + nw] = True
        return torch.where(mask, img * 2.0 - 1.0, torch.full_like(img, -1.0))
    return img * 2.0 - 1.0


@dataclasses.dataclass(frozen=True)
class Pi05ActionOutput:
    actions: torch.Tensor            # [B, horizon, action_dim] fp32
    latency_ms: float                # wall time of the call: pre-processing, prefill, denoise loop, result materialised
    phase_ms: Dict[str, float]


class Pi05Policy:
    def __init__(self) -> None:
        raise RuntimeError("Pi05Policy() is not a public constructor. Use Pi05Policy.from_pretrained(...) or "
                           "Pi05Policy.from_lerobot_policy(...).")

    # ------------------------------------------------------------------ construction
    @classmethod
    def _make(cls, cfg, state_dict, *, dtype, execution, camera_keys=None, n_action_steps=None, action_dim=None):
        self = object.__new__(cls)
        self.config, self._state_dict, self._dtype = cfg, state_dict, dtype
        self._rpu_execution = execution
        chunk = (execution.get("prefill") or {}).get("chunk_size", "auto") if execution else "auto"
        self._vlm_chunk_size = 0 if chunk == "auto" else chunk
        self._engine = None
        self._frozen = False
        self.last_latency_ms = 0.0
        self._prepared: Dict[tuple, bool] = {}
        self.camera_keys = list(camera_keys) if camera_keys else None
        self.n_action_steps = n_action_steps or cfg.horizon
        self.action_dim = action_dim or cfg.action_dim
        self._queue: deque = deque()
        self.default_num_steps = 10
        return self

    @classmethod
    def from_pretrained(cls, pretrained_name_or_path: str, *, dtype: torch.dtype = torch.float16,
                        trust_remote_code: bool = False, vlm_chunk_size: Optional[int] = None, rpu_execution=None,
                        **kw: Any) -> "Pi05Policy":
        ep = "Pi05Policy.from_pretrained"
        if not isinstance(trust_remote_code, bool):
            raise TypeError(f"{ep}: trust_remote_code must be bool, got {trust_remote_code!r}")
        if trust_remote_code is not False:
            raise ValueError(f"{ep} requires trust_remote_code=False; custom model code is not supported.")
        execution = normalize_rpu_execution(rpu_execution, entry_point=ep, vlm_chunk_size=vlm_chunk_size, supported=_STAGES)
        if dtype not in (torch.float16, torch.bfloat16):
            raise RPUUnsupportedDtypeError(f"{ep}: dtype must be torch.float16 or torch.bfloat16, got {dtype}")
        from ..adapters.pi05 import load_checkpoint
        cfg, sd, meta = load_checkpoint(pretrained_name_or_path)
        return cls._make(cfg, sd, dtype=dtype, execution=execution, **meta)

    @classmethod
    def from_lerobot_policy(cls, lerobot_policy: Any, *, rpu_execution=None) -> "Pi05Policy":
        execution = normalize_rpu_execution(rpu_execution, entry_point="Pi05Policy.from_lerobot_policy", supported=_STAGES)
        from ..adapters.pi05 import config_from_lerobot
        model = getattr(lerobot_policy, "model", lerobot_policy)
        cfg, meta = config_from_lerobot(getattr(lerobot_policy, "config", None), model)
        sd = {k: v.detach() for k, v in model.state_dict().items()}
        dtypes = {v.dtype for v in sd.values() if v.is_floating_point()}
        dtype = torch.bfloat16 if dtypes == {torch.bfloat16} else torch.float16
        return cls._make(cfg, sd, dtype=dtype, execution=execution, **meta)

    @classmethod
    def from_state_dict(cls, cfg, state_dict, *, dtype=torch.float16, rpu_execution=None, **meta) -> "Pi05Policy":
        """Build from an in-memory configuration and weights (synthetic benchmarks, tests)."""
        execution = normalize_rpu_execution(rpu_execution, entry_point="Pi05Policy.from_state_dict", supported=_STAGES)
        return cls._make(cfg, state_dict, dtype=dtype, execution=execution, **meta)

    # ------------------------------------------------------------------ device
    def to(self, device: Any, *, max_batch: int = 1) -> "Pi05Policy":
        name = str(device).lower()
        if name.startswith(("rpu", "cuda")):
            if self._engine is None:
                from ..models.pi05 import Pi05Engine
                from ..runtime import live_handle
                live_handle.claim(self)
                try:
                    self._engine = Pi05Engine(self.config, self._state_dict, dtype=self._dtype, max_batch=max_batch)
                except Exception as e:  # noqa: BLE001
                    live_handle.poison(self, f"Pi0.5 install failed: {type(e).__name__}: {e}")
                    raise
                self._state_dict = None
            elif max_batch > self._engine.max_batch:
                raise RPUBackendError("the policy was installed with a smaller max_batch; reload to grow it")
            return self
        if self._engine is not None:
            raise RPUBackendError("this policy's weights were packed for the accelerator exactly once; reload the "
                                  "checkpoint to run it elsewhere")
        return self

    @property
    def engine(self):
        if self._engine is None:
            raise RPUBackendError("call policy.to('rpu') before running the policy")
        return self._engine

    # ------------------------------------------------------------------ batch plumbing
    def _inputs(self, batch: dict):
        cfg = self.config
        keys = self.camera_keys or sorted(k for k in batch if k.startswith(IMAGE_PREFIX))
        present = [k for k in keys if k in batch and batch[k] is not None]
        if not present:
            raise RPUBackendError(f"batch has no image under any of {keys or [IMAGE_PREFIX + '<camera>']}")
        if TOKENS_KEY not in batch:
            raise RPUBackendError(f"batch needs {TOKENS_KEY!r} (and {TOKEN_MASK_KEY!r}): run the policy pre-processor")
        tokens = torch.as_tensor(batch[TOKENS_KEY])
        tokens = tokens if tokens.dim() == 2 else tokens[None]
        B = tokens.shape[0]
        tmask = torch.as_tensor(batch.get(TOKEN_MASK_KEY, torch.ones_like(tokens))).bool().reshape(B, -1)
        if tokens.shape[1] > cfg.max_lang_tokens:
            raise RPUBackendError(f"{tokens.shape[1]} language tokens exceed the installed maximum {cfg.max_lang_tokens}")
        views, vmask = [], []
        dev = self.engine.device
        for k in keys[:cfg.num_views]:
            if k in present:
                im = torch.as_tensor(batch[k]).to(dev, torch.float32)
                im = im if im.dim() == 4 else im[None]
                views.append(resize_with_pad(im, cfg.vision.image_size))
                vmask.append(torch.ones(B, dtype=torch.bool))
            else:
                views.append(torch.full((B, 3, cfg.vision.image_size, cfg.vision.image_size), -1.0, device=dev))
                vmask.append(torch.zeros(B, dtype=torch.bool))
        while len(views) < cfg.num_views:
            views.append(torch.full_like(views[0], -1.0))
            vmask.append(torch.zeros(B, dtype=torch.bool))
        images = torch.stack(views, 1)
        noise = batch.get("noise")
        if noise is None:
            noise = torch.randn(B, cfg.horizon, cfg.action_dim, device=dev, dtype=torch.float32)
        return images, torch.stack(vmask, 1), tokens, tmask, torch.as_tensor(noise)

    # ------------------------------------------------------------------ public runs
    @torch.no_grad()
    def prepare_graphs(self, batch: dict, num_steps: Optional[int] = None) -> dict:
        """BUILD the denoise graph for this batch geometry, REPLAY it once, check that both runs agree
        bit for bit, then freeze: later calls may only use prepared ``(batch size, num_steps)`` pairs."""
        ep = "Pi05Policy.prepare_graphs"
        batch = _validate_batch(batch, entry_point=ep)
        steps = _validate_num_steps(num_steps, entry_point=ep) or self.default_num_steps
        eng = self.engine
        args = self._inputs(batch)
        key = (args[0].shape[0], steps)
        eng._graphs.pop(key, None)
        eng._prefill_graphs.clear()                       # vision + prefix prefill graph of this geometry is rebuilt too
        a = eng.predict(*args, num_steps=steps).clone()   # BUILD: prefill graph (vision tower + prefix) and denoise graph
        b = eng.predict(*args, num_steps=steps).clone()   # REPLAY of both
        eng.check_status()
        if not torch.equal(a, b):
            raise RPUBackendError("Pi0.5 graph BUILD and REPLAY disagree: the captured stages are not deterministic")
        self._prepared[key] = True
        self._frozen = True
        return {"batch_size": key[0], "num_steps": steps, "graphs": len(eng._graphs) + len(eng._prefill_graphs),
                "stages": ["vision+prefix", "denoise"], "deterministic": True}

    @torch.no_grad()
    def predict_action_chunk(self, batch: dict, num_steps: Optional[int] = None) -> torch.Tensor:
        ep = "Pi05Policy.predict_action_chunk"
        batch = _validate_batch(batch, entry_point=ep)
        steps = _validate_num_steps(num_steps, entry_point=ep) or self.default_num_steps
        args = self._inputs(batch)
        if self._frozen and (args[0].shape[0], steps) not in self._prepared:
            raise RPUBackendError(f"{ep}: graphs are frozen for {sorted(self._prepared)}; (batch, num_steps)="
                                  f"{(args[0].shape[0], steps)} was not prepared")
        # RPU_PI05_FUSED_DENOISE=0 / RPU_PI05_DENOISE_UNROLL=0: launch the Euler steps one by one instead of replaying the
        # whole loop from one captured graph (debugging and A/B timing)
        from ..runtime.control import rpu_env_bool
        one_graph = rpu_env_bool("RPU_PI05_FUSED_DENOISE", True) and rpu_env_bool("RPU_PI05_DENOISE_UNROLL", True)
        import time
        t0 = time.perf_counter()
        out = self.engine.predict(*args, num_steps=steps, use_graph=one_graph)
        out = out[:, :, :self.action_dim].float().clone()
        if out.is_cuda:
            torch.cuda.current_stream(out.device).synchronize()
        self.last_latency_ms = (time.perf_counter() - t0) * 1000.0       # device work of the chunk, result materialised
        return out

    @torch.no_grad()
    def infer(self, batch: dict, num_steps: Optional[int] = None) -> "Pi05ActionOutput":
        """``predict_action_chunk`` with the wall time of the call attached (pre-processing included)."""
        import time
        t0 = time.perf_counter()
        actions = self.predict_action_chunk(batch, num_steps)
        return Pi05ActionOutput(actions=actions, latency_ms=(time.perf_counter() - t0) * 1000.0,
                                phase_ms={"device_ms": self.last_latency_ms})

    @torch.no_grad()
    def select_action(self, batch: dict) -> torch.Tensor:
        """Next action ``[B, action_dim]``; refills the queue with a fresh chunk when it runs dry."""
        batch = _validate_batch(batch, entry_point="Pi05Policy.select_action")
        if not self._queue:
            chunk = self.predict_action_chunk(batch)[:, :self.n_action_steps].cpu()
            self._queue.extend(chunk.transpose(0, 1))
        return self._queue.popleft()

    def reset(self) -> None:
        self._queue.clear()

    def close(self) -> None:
        if self._engine is not None:
            self._engine.close()
            self._engine = None


__all__ = ["Pi05Policy", "Pi05ActionOutput", "resize_with_pad"]
