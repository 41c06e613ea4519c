"""``RPUModelForCausalLM``: the loader entry point for decoder-only language models.

``from_pretrained(path, dtype=..., device=None|"rpu", rpu_execution=None, **hf_kwargs)``:
every rejection -- execution config, dtype, reserved Hugging Face kwargs, ``trust_remote_code``,
architecture routing, the adapter's profile allow-list -- happens from the config alone, before a
single weight is read.  With ``device="rpu"`` the weights stream from the safetensors shards
straight into the packed device layout and the runtime handle is returned; with ``device=None``
the Hugging Face model is loaded on the CPU with an adapter-bound ``.to("rpu")``.
Reference: ``python/rpu_backend/api/causal_lm.py:155-278``.
"""
from __future__ import annotations

import os

import torch

from ..runtime import live_handle
from ..runtime.registry import get_adapter
from ._execution import normalize_rpu_execution
from ._loading import checkpoint_tensor_getter, resolve_config_architecture, resolve_loader_device
from .errors import RPUUnsupportedDtypeError, UnsupportedModelError

_claim_live_instance = live_handle.claim
_poison_live_instance = live_handle.poison


class RPUModelForCausalLM:
    """Stateless entry point; not a subclass of any Hugging Face class."""

    _RESERVED_HF_KWARGS = frozenset({"torch_dtype", "dtype", "device_map", "device", "low_cpu_mem_usage", "tp_plan",
                                     "load_in_8bit", "load_in_4bit", "quantization_config"})
    _SUPPORTED_BUILTIN_ARCHITECTURES = frozenset({"LlamaForCausalLM", "Qwen3ForCausalLM"})
    _CONFIG_KWARGS = frozenset({"cache_dir", "revision", "subfolder", "local_files_only", "token", "force_download",
                                "proxies"})
    SUPPORTED_DTYPES = (torch.float16, torch.bfloat16)

    @classmethod
    def from_pretrained(cls, hf_repo_or_path: str, *, dtype: torch.dtype = torch.float16, device=None,
                        rpu_execution=None, max_batch: int = 64, tp=None, **hf_kwargs):
        ep = "RPUModelForCausalLM.from_pretrained"
        execution = normalize_rpu_execution(rpu_execution, entry_point=ep,
                                            supported={"prefill": ("chunk_size", "padding_rows", "padding_budget")})
        if dtype not in cls.SUPPORTED_DTYPES:
            raise RPUUnsupportedDtypeError(f"the kernels take torch.float16 or torch.bfloat16, got {dtype}. Load the "
                                           "CPU reference separately if you need an fp32 baseline for comparison.")
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
        arch = resolve_config_architecture(config, source=hf_repo_or_path, entry_point=ep,
                                           supported_builtins=cls._SUPPORTED_BUILTIN_ARCHITECTURES)
        adapter_cls = get_adapter(arch)
        if hasattr(adapter_cls, "preflight"):
            adapter_cls.preflight(config)
        if hasattr(adapter_cls, "preflight_execution"):
            adapter_cls.preflight_execution(config, execution)

        from ..quant.load import is_w8a16_config, load_w8a16_model
        if to_rpu and os.path.isdir(hf_repo_or_path):
            # streamed load: safetensors -> packed device weights, no host-side model object
            from ..quant.load import is_w4a16_config, w4a16_tensor_getter, w8a16_tensor_getter
            get = (w8a16_tensor_getter(hf_repo_or_path, config) if is_w8a16_config(config)
                   else w4a16_tensor_getter(hf_repo_or_path, config) if is_w4a16_config(config)
                   else checkpoint_tensor_getter(hf_repo_or_path))
            adapter = adapter_cls(None, config=config, get_weight=get, rpu_execution=execution, dtype=dtype)
            return adapter.to_rpu(max_batch=max_batch, tp=tp)
        if is_w8a16_config(config):
            model = load_w8a16_model(config, hf_repo_or_path, dtype=dtype, **cfg_kwargs)
        else:
            from transformers import AutoModelForCausalLM
            model = AutoModelForCausalLM.from_pretrained(hf_repo_or_path, dtype=dtype, trust_remote_code=False,
                                                         **hf_kwargs)
        model.eval()
        model._rpu_execution = execution
        adapter = adapter_cls(model, dtype=dtype)
        adapter._rpu_execution = execution
        if to_rpu:
            return adapter.to_rpu(max_batch=max_batch, tp=tp)
        return model


__all__ = ["RPUModelForCausalLM"]
