"""``RPUModelForConditionalGeneration``: loader entry point for vision-language models.

Only ``Qwen3VLForConditionalGeneration`` is routed here.  As for the causal-LM loader, every rejection
(execution config, dtype, reserved kwargs, ``trust_remote_code``, architecture, profile) is decided from
the config before any weight is read.  Reference: ``python/rpu_backend/api/conditional_generation.py:58-170``.
"""
from __future__ import annotations

import os

import torch

from ._execution import normalize_rpu_execution
from ._loading import checkpoint_tensor_getter, resolve_loader_device
from .errors import RPUUnsupportedDtypeError, UnsupportedModelError


class RPUModelForConditionalGeneration:
    _RESERVED_HF_KWARGS = frozenset({"torch_dtype", "dtype", "device_map", "device", "low_cpu_mem_usage", "tp_plan",
                                     "load_in_8bit", "load_in_4bit", "quantization_config"})
    _SUPPORTED_ARCHITECTURES = frozenset({"Qwen3VLForConditionalGeneration"})
    _CONFIG_KWARGS = frozenset({"cache_dir", "revision", "subfolder", "local_files_only", "token", "force_download",
                                "proxies"})
    SUPPORTED_DTYPES = (torch.float16, torch.bfloat16)

    @classmethod
    def from_pretrained(cls, hf_repo_or_path: str, *, dtype: torch.dtype = torch.float16, device=None,
                        rpu_execution=None, max_seq_len: int = 4096, max_patches: int = 4096, tp=None, **hf_kwargs):
        ep = "RPUModelForConditionalGeneration.from_pretrained"
        execution = normalize_rpu_execution(rpu_execution, entry_point=ep,
                                            supported={"prefill": ("chunk_size", "padding_rows", "padding_budget"),
                                                       "vision": ("chunk_size",)})
        if dtype not in cls.SUPPORTED_DTYPES:
            raise RPUUnsupportedDtypeError(f"the kernels take torch.float16 or torch.bfloat16, got {dtype}")
        clash = cls._RESERVED_HF_KWARGS & set(hf_kwargs)
        if clash:
            raise ValueError(f"{ep}: hf_kwargs cannot include reserved key(s) {sorted(clash)}; the library manages "
                             "these internally. Remove these keys from your call.")
        if hf_kwargs.pop("trust_remote_code", False) is not False:
            raise ValueError(f"{ep} requires trust_remote_code=False; custom model code is not supported.")
        to_rpu = resolve_loader_device(device, entry_point=ep)
        from transformers import AutoConfig
        cfg_kwargs = {k: v for k, v in hf_kwargs.items() if k in cls._CONFIG_KWARGS}
        try:
            config = AutoConfig.from_pretrained(hf_repo_or_path, trust_remote_code=False, **cfg_kwargs)
        except (OSError, ValueError) as e:
            raise UnsupportedModelError(f"Could not load HF config for {hf_repo_or_path!r}: {type(e).__name__}: {e}.") from e
        archs = getattr(config, "architectures", None) or []
        if not archs or archs[0] not in cls._SUPPORTED_ARCHITECTURES:
            raise UnsupportedModelError(f"{ep} supports {sorted(cls._SUPPORTED_ARCHITECTURES)}; got architectures={archs!r}")
        from ..adapters.qwen3_vl import Qwen3VLAdapter
        Qwen3VLAdapter.preflight(config)
        Qwen3VLAdapter.preflight_execution(config, execution)
        if to_rpu and os.path.isdir(hf_repo_or_path):
            from ..quant.load import is_w8a16_config, w8a16_tensor_getter
            get = (w8a16_tensor_getter(hf_repo_or_path, config) if is_w8a16_config(config)
                   else checkpoint_tensor_getter(hf_repo_or_path))
            adapter = Qwen3VLAdapter(None, config=config, get_weight=get, rpu_execution=execution, dtype=dtype)
            return adapter.to_rpu(max_seq_len=max_seq_len, max_patches=max_patches, tp=tp)
        from transformers import AutoModelForImageTextToText
        model = AutoModelForImageTextToText.from_pretrained(hf_repo_or_path, dtype=dtype, trust_remote_code=False, **hf_kwargs)
        model.eval()
        model._rpu_execution = execution
        adapter = Qwen3VLAdapter(model, rpu_execution=execution, dtype=dtype)
        if to_rpu:
            return adapter.to_rpu(max_seq_len=max_seq_len, max_patches=max_patches, tp=tp)
        model.to_rpu = adapter.to_rpu
        return model


__all__ = ["RPUModelForConditionalGeneration"]
