"""Shared adapter logic of the decoder-only families (Qwen3, Llama).

An adapter (1) rejects unsupported configurations from the config alone, before any weight is
read (``preflight`` / ``preflight_execution``), (2) claims the process-wide live-handle slot,
(3) packs the weights for the accelerator exactly once and (4) returns the runtime handle.
Reference flow: ``python/rpu_backend/adapters/qwen3.py:253-288,411-556``.
"""
from __future__ import annotations

import threading
from typing import Callable, FrozenSet, Optional, Tuple

import torch

from ..api._execution import bind_rpu_execution, prefill_chunk_rows
from ..api.errors import (RPUBackendError, RPUUnsupportedDtypeError, UnsupportedModelError,
                          WeightShapeMismatchError)
from ..models.decoder import DecoderConfig
from ..runtime import live_handle
from ..runtime.control import rpu_env_exact1

_PACK_LOCK = threading.Lock()
Profile = Tuple[int, int, int, int]


def config_profile(config) -> Profile:
    return (int(config.hidden_size), int(config.intermediate_size), int(config.num_hidden_layers),
            int(config.num_key_value_heads))


def config_is_w8a16(config) -> bool:
    qc = getattr(config, "quant_config", None)
    return isinstance(qc, dict) and qc.get("method") == "w8a16"


class CausalLMAdapter:
    ARCH: str = ""
    FAMILY: str = ""
    SUPPORTED_PROFILES: FrozenSet[Profile] = frozenset()
    W8A16_ONLY_PROFILES: FrozenSet[Profile] = frozenset()
    UNLISTED_GATE: str = ""           # env var (exact literal 1) admitting an unlisted profile for evaluation
    SUPPORTED_EXECUTION = {"prefill": ("chunk_size", "padding_rows", "padding_budget")}

    # ---- config-only checks -------------------------------------------------------------------
    @classmethod
    def check_profile(cls, config) -> None:
        profile = config_profile(config)
        if profile in cls.W8A16_ONLY_PROFILES:
            qc = getattr(config, "quant_config", None) or {}
            exact = (config_is_w8a16(config) and qc.get("quantized_lm_head") is True
                     and qc.get("lm_head_untied") is True and qc.get("quantized_embed_tokens") is False)
            if not exact:
                raise UnsupportedModelError(f"{cls.FAMILY} profile {profile} requires the release W8A16 profile with "
                                            "an untied INT8 lm_head and FP16 embeddings.")
            return
        if profile in cls.SUPPORTED_PROFILES:
            return
        if cls.UNLISTED_GATE and rpu_env_exact1(cls.UNLISTED_GATE):
            return
        raise UnsupportedModelError(
            f"{cls.FAMILY} with profile (hidden_size={profile[0]}, intermediate_size={profile[1]}, "
            f"num_hidden_layers={profile[2]}, num_key_value_heads={profile[3]}) has no admitted execution profile in "
            f"this build (deny by default). Supported fp16 profiles: {sorted(cls.SUPPORTED_PROFILES)}. "
            f"W8A16-only profiles: {sorted(cls.W8A16_ONLY_PROFILES)}.")

    @classmethod
    def preflight(cls, config) -> None:
        cls.check_profile(config)
        hd = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        if hd not in (64, 128, 256):
            raise UnsupportedModelError(f"{cls.FAMILY}: head_dim {hd} is not one of 64/128/256")

    @classmethod
    def preflight_execution(cls, config, execution) -> None:
        chunk = (execution or {}).get("prefill", {}).get("chunk_size", "auto") if execution else "auto"
        if chunk != "auto" and chunk > 65536:
            raise RPUBackendError(f"{cls.FAMILY}: prefill chunk_size {chunk} exceeds the 65536-row ceiling")

    # ---- instance ---------------------------------------------------------------------------------
    def __init__(self, model=None, *, config=None, get_weight: Optional[Callable[[str], torch.Tensor]] = None,
                 rpu_execution=None, dtype: torch.dtype = torch.float16):
        """Bind to a loaded Hugging Face model, or to ``(config, get_weight)`` for streamed loading."""
        self.model = model
        self.config = config if config is not None else model.config
        self.check_profile(self.config)
        self._get_weight = get_weight
        self._dtype = dtype
        self._handle = None
        owner = model if model is not None else self
        bind_rpu_execution(owner, rpu_execution, entry_point=f"{type(self).__name__}", supported=self.SUPPORTED_EXECUTION)
        self._rpu_execution = owner._rpu_execution
        if model is not None:
            self._install_to_hook(model)

    def _install_to_hook(self, model) -> None:
        """Instance-level ``.to('rpu')`` interception: everything else goes to ``nn.Module.to``."""
        adapter = self
        plain_to = model.to

        def to(device=None, *a, **kw):
            if device is not None and str(device).lower().startswith(("rpu",)):
                return adapter.to_rpu()
            return plain_to(device, *a, **kw)

        model.to = to

    def decoder_config(self) -> DecoderConfig:
        return DecoderConfig.from_hf(self.config)

    def _weights(self) -> Callable[[str], torch.Tensor]:
        if self._get_weight is not None:
            return self._get_weight
        sd = self.model.state_dict()

        def get(name: str) -> torch.Tensor:
            if name == "lm_head.weight" and name not in sd:
                return sd["model.embed_tokens.weight"]
            return sd[name]

        get.names = frozenset(sd)  # type: ignore[attr-defined]
        get.scale = lambda n: sd.get(n[:-len(".weight")] + ".weight_scale")  # type: ignore[attr-defined]
        return get

    def to_rpu(self, *, max_batch: int = 64, tp=None):
        """Pack the weights once, create the native runtime and return the runtime handle."""
        if self._handle is not None:
            return self._handle
        if self._dtype not in (torch.float16, torch.bfloat16):
            raise RPUUnsupportedDtypeError(f"kernels take float16 or bfloat16, got {self._dtype}")
        if not _PACK_LOCK.acquire(blocking=False):
            raise RPUBackendError("another model is being packed for the accelerator in this process")
        try:
            owner = self.model if self.model is not None else self
            live_handle.claim(owner)
            from ..runtime.causal_lm import RPUCausalLM
            from ..runtime.engine import DecoderEngine
            cfg = self.decoder_config()
            get = self._weights()
            self._validate_shapes(cfg, get)
            chunk = prefill_chunk_rows(self._rpu_execution)
            quant = "w8a16" if config_is_w8a16(self.config) else None
            try:
                engine = DecoderEngine(cfg, get, dtype=self._dtype, max_batch=max_batch, max_seq_len=16,
                                       max_prefill_tokens=chunk, tp=tp, quant=quant)
            except Exception as e:
                live_handle.poison(owner, f"{type(self).__name__}.to_rpu failed after weight packing began: {e}")
                raise
            self._handle = RPUCausalLM(engine, self.config, execution=self._rpu_execution, owner=self.model)
            live_handle.rebind(owner, self._handle)
            return self._handle
        finally:
            _PACK_LOCK.release()

    def _validate_shapes(self, cfg: DecoderConfig, get) -> None:
        names = getattr(get, "names", None)
        if names is None:
            return
        need = ["model.embed_tokens.weight", "model.norm.weight", "model.layers.0.self_attn.q_proj.weight"]
        missing = [n for n in need if n not in names]
        if missing:
            raise WeightShapeMismatchError(f"checkpoint is missing {missing}")


__all__ = ["CausalLMAdapter", "config_profile", "config_is_w8a16"]
