"""Qwen3-VL adapter: profile guard, then vision tower + M-RoPE text engine on the accelerator.

Reference: ``python/rpu_backend/adapters/qwen3_vl/__init__.py:90-121,541`` (admitted text and vision
profiles, adapter class), ``adapters/qwen3_vl/vision.py``, ``adapters/qwen3_vl/text.py``.
"""
from __future__ import annotations

import os
from typing import Callable, Optional

import torch

from ...models import qwen3_vl as Q
from ...runtime import live_handle
from ...runtime.errors import RPUBackendError, UnsupportedModelError



class Qwen3VLAdapter:
    ARCHITECTURE = "Qwen3VLForConditionalGeneration"
    EXECUTION_STAGES = {"prefill": ("chunk_size", "padding_rows", "padding_budget"), "vision": ("chunk_size",)}

    @classmethod
    def preflight(cls, config) -> None:
        Q.preflight(config, strict=os.environ.get("RPU_QWEN3_VL_ALLOW_ANY_PROFILE", "0") != "1")
        from ...runtime.control import rpu_env_exact1
        prof32 = Q.TEXT_PROFILES.get(Q.text_config_of(config).profile()) == "qwen3-vl-32b"
        if prof32 and not rpu_env_exact1("QWEN3_VL_32B_ALLOW_GRAPH_BLOCKED"):
            # fail-closed evaluation gate: the 32B profile has not been run end to end on this backend
            raise UnsupportedModelError("the Qwen3-VL 32B profile is evaluation-gated: set QWEN3_VL_32B_ALLOW_GRAPH_BLOCKED=1 "
                                        "(exactly 1) to admit it")
        from ..causal_base import config_is_w8a16
        if config_is_w8a16(config):
            prof = Q.text_config_of(config).profile()
            if Q.TEXT_PROFILES.get(prof) != "qwen3-vl-32b":
                raise UnsupportedModelError("W8A16 Qwen3-VL is admitted for the 32B text profile only")

    @classmethod
    def preflight_execution(cls, config, execution) -> None:
        for stage in (execution or {}):
            if stage not in cls.EXECUTION_STAGES:
                raise UnsupportedModelError(f"Qwen3-VL has no execution stage {stage!r}")

    def __init__(self, model=None, *, config=None, get_weight: Optional[Callable[[str], torch.Tensor]] = None,
                 rpu_execution=None, dtype=torch.float16, names=None):
        if model is None and (config is None or get_weight is None):
            raise RPUBackendError("Qwen3VLAdapter needs a model, or a config and a weight getter")
        self.model, self.config = model, config if config is not None else model.config
        self._get, self._names = get_weight, names
        self._rpu_execution, self.dtype = rpu_execution, dtype
        self.preflight(self.config)

    def _weights(self):
        if self._get is not None:
            return self._get, (self._names or getattr(self._get, "names", None))
        sd = self.model.state_dict()
        return (lambda n: sd[n]), set(sd)

    def to_rpu(self, *, max_seq_len: int = 4096, max_patches: int = 4096, tp=None):
        from ...runtime.conditional_generation import RPUConditionalGeneration
        ex = self._rpu_execution or {}
        chunk = (ex.get("prefill") or {}).get("chunk_size", "auto")
        max_prefill = 4096 if chunk in ("auto", None) else int(chunk)
        quant = "w8a16" if getattr(self.config, "quant_config", None) else None
        get, names = self._weights()
        token = live_handle.claim(self)
        try:
            eng = Q.Qwen3VLEngine(self.config, get, dtype=self.dtype, max_seq_len=max_seq_len, max_patches=max_patches,
                                  max_prefill_tokens=min(max_prefill, max_seq_len), tp=tp, quant=quant,
                                  names=None if names is None else set(names))
        except Exception as e:  # noqa: BLE001
            live_handle.poison(self, f"Qwen3-VL install failed: {type(e).__name__}: {e}")
            raise
        handle = RPUConditionalGeneration(eng, self.config, execution=self._rpu_execution)
        live_handle.rebind(self, handle)
        self.model = None          # the host copy is not kept: weights live in the packed device layout
        return handle


__all__ = ["Qwen3VLAdapter"]
