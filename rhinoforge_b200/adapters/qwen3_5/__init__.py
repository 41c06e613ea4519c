"""Qwen3.5 adapter (hybrid full-attention + Gated-DeltaNet decoder).

    model = Qwen3_5Adapter(hf_model, rpu_execution=cfg).to_rpu(max_seq_len=L)
    cache = Qwen3_5Cache.from_config(text_config, max_seq_len=L)
    out = model.generate(ids, past_key_values=cache, max_new_tokens=n, do_sample=False)

Dense text profiles only (mixture-of-experts variants are rejected); the prefill chunk size must be a
multiple of 64.  Reference: ``python/rpu_backend/adapters/qwen3_5/__init__.py:49-56,141-160,182,205-212,313``.
"""
from __future__ import annotations

import os
from typing import Callable, Optional

import torch

from ...models.decoder import DecoderConfig
from ...runtime import live_handle
from ...runtime.errors import RPUBackendError, RPUConfigError, UnsupportedModelError

PROFILES = {(1024, 3584, 24, 2): "qwen3.5-0.8b", (2048, 6144, 24, 2): "qwen3.5-2b", (2560, 9216, 32, 4): "qwen3.5-4b",
            (4096, 12288, 32, 4): "qwen3.5-9b"}


def _text(config):
    return getattr(config, "text_config", config)


class Qwen3_5Adapter:
    ARCHITECTURE = "Qwen3_5ForConditionalGeneration"
    EXECUTION_STAGES = {"prefill": ("chunk_size", "padding_rows", "padding_budget"), "vision": ("chunk_size",)}

    @classmethod
    def preflight(cls, config) -> None:
        tc = _text(config)
        if getattr(tc, "num_experts", 0) or "moe" in str(getattr(tc, "model_type", "")):
            raise UnsupportedModelError("Qwen3.5 mixture-of-experts checkpoints are not supported")
        cfg = DecoderConfig.from_hf(tc)
        if cfg.layer_types is None:
            raise UnsupportedModelError("Qwen3.5 config carries no layer_types")
        vc = getattr(config, "vision_config", None)
        if vc is not None and getattr(config, "rpu_use_vision", False):
            # the tower is the Qwen3-VL ViT without DeepStack taps: anything else is another architecture
            if tuple(getattr(vc, "deepstack_visual_indexes", ()) or ()):
                raise UnsupportedModelError("a Qwen3.5 vision tower has no DeepStack taps; this config lists "
                                            f"{list(vc.deepstack_visual_indexes)}")
            if getattr(vc, "hidden_act", "gelu_pytorch_tanh") not in ("gelu_pytorch_tanh", "gelu"):
                raise UnsupportedModelError("Qwen3.5 vision activation must be gelu_pytorch_tanh or gelu")
        if cfg.gdn_dk != 128 or cfg.gdn_dv % 32 or cfg.gdn_conv != 4:
            raise UnsupportedModelError(f"Qwen3.5 linear-attention geometry (Dk={cfg.gdn_dk}, Dv={cfg.gdn_dv}, "
                                        f"conv={cfg.gdn_conv}) is not built (Dk 128, Dv multiple of 32, conv 4)")
        if os.environ.get("RPU_QWEN3_5_ALLOW_ANY_PROFILE", "0") != "1" and cfg.profile() not in PROFILES:
            raise UnsupportedModelError(f"Qwen3.5 profile {cfg.profile()} is not admitted; known: {sorted(PROFILES)}")

    @classmethod
    def preflight_execution(cls, config, execution) -> None:
        for stage, fields in (execution or {}).items():
            if stage not in cls.EXECUTION_STAGES:
                raise RPUConfigError(f"Qwen3.5 has no execution stage {stage!r}")
            chunk = fields.get("chunk_size")
            if stage == "prefill" and isinstance(chunk, int) and chunk % 64:
                raise RPUConfigError(f"Qwen3.5 prefill chunk_size must be a multiple of 64, got {chunk}")

    def __init__(self, model=None, *, config=None, get_weight: Optional[Callable[[str], torch.Tensor]] = None,
                 rpu_execution=None, dtype=torch.float16):
        if model is None and (config is None or get_weight is None):
            raise RPUBackendError("Qwen3_5Adapter needs a model, or a config and a weight getter")
        self.model, self.config = model, config if config is not None else model.config
        self._get, self._rpu_execution, self.dtype = get_weight, rpu_execution, dtype
        self.preflight(self.config)
        self.preflight_execution(self.config, rpu_execution)
        if model is not None:
            self._install_to_hook(model)

    def _install_to_hook(self, model) -> None:
        orig = model.to

        def to(device=None, *a, **kw):
            if str(device).lower().startswith(("rpu", "cuda")):
                return self.to_rpu()
            return orig(device, *a, **kw)
        try:
            model.to = to
        except Exception:  # noqa: BLE001
            pass

    def _weights(self):
        if self._get is not None:
            get, names = self._get, getattr(self._get, "names", None)
        else:
            sd = self.model.state_dict()
            get, names = (lambda n: sd[n]), set(sd)
        nested = names is not None and any(n.startswith("model.language_model.") for n in names)

        def text_get(name: str) -> torch.Tensor:
            if nested and name.startswith("model."):
                return get("model.language_model." + name[len("model."):])
            return get(name)
        if names is not None:
            text_get.names = {("model." + n[len("model.language_model."):]) if n.startswith("model.language_model.") else n
                              for n in names}
        return text_get

    def to_rpu_vision(self, *, max_seq_len: int = 8192, max_patches: int = 4096, tp=None):
        """The multimodal handle: vision tower + hybrid decoder (``config.rpu_use_vision`` selects it in :meth:`to_rpu`).
        The tower is the Qwen3-VL ViT without DeepStack (reference: ``python/rpu_backend/adapters/qwen3_5/vision.py:1-30``),
        so the Qwen3-VL engine serves it: image rows are spliced into the embeddings and the text runs under three-axis
        M-RoPE positions; the Gated-DeltaNet layers see the image rows as ordinary tokens."""
        from ...models.qwen3_vl import Qwen3VLEngine
        from ...runtime.conditional_generation import RPUConditionalGeneration
        if getattr(self.config, "vision_config", None) is None:
            raise UnsupportedModelError("this Qwen3.5 checkpoint has no vision_config")
        if self._get is not None:
            get, names = self._get, getattr(self._get, "names", None)
        else:
            sd = self.model.state_dict()
            get, names = (lambda n: sd[n]), set(sd)
        ex = self._rpu_execution or {}
        chunk = (ex.get("prefill") or {}).get("chunk_size", "auto")
        max_prefill = min(max_seq_len, 8192) if chunk in ("auto", None) else int(chunk)
        live_handle.claim(self)
        try:
            eng = Qwen3VLEngine(self.config, get, dtype=self.dtype, max_seq_len=max_seq_len, max_patches=max_patches,
                                max_prefill_tokens=max_prefill, tp=tp, names=None if names is None else set(names))
        except Exception as e:  # noqa: BLE001
            live_handle.poison(self, f"Qwen3.5 install failed: {type(e).__name__}: {e}")
            raise
        handle = RPUConditionalGeneration(eng, self.config, execution=self._rpu_execution)
        live_handle.rebind(self, handle)
        self.model = None
        return handle

    def to_rpu(self, *, max_seq_len: int = 8192, max_batch: int = 1, tp=None, **kw):
        if getattr(self.config, "vision_config", None) is not None and getattr(self.config, "rpu_use_vision", False):
            return self.to_rpu_vision(max_seq_len=max_seq_len, tp=tp, **kw)
        from ...runtime.causal_lm import RPUCausalLM
        from ...runtime.engine import DecoderEngine
        cfg = DecoderConfig.from_hf(_text(self.config))
        ex = self._rpu_execution or {}
        from ...runtime.control import rpu_env_int
        chunk = (ex.get("prefill") or {}).get("chunk_size", "auto")
        if chunk in ("auto", None):
            env_chunk = rpu_env_int("QWEN3_5_TEXT_CHUNK", 0)          # process-wide default when the config says auto
            if env_chunk % 64:
                raise RPUConfigError(f"QWEN3_5_TEXT_CHUNK must be a multiple of 64, got {env_chunk}")
            chunk = env_chunk or "auto"
        self.padding_budget = (ex.get("prefill") or {}).get("padding_budget",
                                                            rpu_env_int("QWEN3_5_TEXT_PADDING_BUDGET", 64))
        max_prefill = min(max_seq_len, 8192) if chunk in ("auto", None) else int(chunk)
        live_handle.claim(self)
        try:
            kw = dict(tp=tp) if tp is not None else {}
            eng = DecoderEngine(cfg, self._weights(), dtype=self.dtype, max_batch=max_batch, max_seq_len=max_seq_len,
                                max_prefill_tokens=max_prefill, **kw)
        except Exception as e:  # noqa: BLE001
            live_handle.poison(self, f"Qwen3.5 install failed: {type(e).__name__}: {e}")
            raise
        handle = RPUCausalLM(eng, self.config, execution=self._rpu_execution, owner=self.model)
        live_handle.rebind(self, handle)
        if os.environ.get("RPU_QWEN3_5_FREE_HF_WEIGHTS", "0") == "1":
            self.model = None
        return handle


__all__ = ["Qwen3_5Adapter", "PROFILES"]
