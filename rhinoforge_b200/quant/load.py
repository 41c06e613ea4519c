"""Loading W8A16 checkpoints (layout written by :mod:`rhinoforge_b200.quant.convert_qwen3`).

Two consumers:

* :func:`w8a16_tensor_getter` -- the streamed path used by ``from_pretrained(device="rpu")``:
  int8 weights and their ``.weight_scale`` siblings go from the safetensors shards straight
  into the engine's packer; nothing is dequantised and no host model object is created.
* :func:`load_w8a16_model` -- the CPU path: a Hugging Face skeleton built on the ``meta`` device
  whose quantised ``nn.Linear`` modules keep int8 ``weight`` Parameters and gain a
  ``weight_scale`` buffer (reference behaviour: ``python/rpu_backend/quant/load.py:227-357``).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, List

import torch
from torch import nn

from .convert_qwen3 import EMBED, LM_HEAD, PROJECTION_SUFFIXES, scale_name

W8A16_METHOD = "w8a16"


def is_w8a16_config(config) -> bool:
    qc = getattr(config, "quant_config", None)
    if qc is None and isinstance(config, dict):
        qc = config.get("quant_config")
    return isinstance(qc, dict) and qc.get("method") == W8A16_METHOD


def is_w4a16_config(config) -> bool:
    qc = getattr(config, "quant_config", None)
    if qc is None and isinstance(config, dict):
        qc = config.get("quant_config")
    return isinstance(qc, dict) and qc.get("method") == "w4a16"


# The one image-text profile admitted in W8A16: Qwen3-VL-32B with the decoder projections quantised, the lm_head, the
# embeddings and the whole vision tower left in 16 bits (reference: ``python/rpu_backend/quant/load.py:29-103``).
QWEN3_VL_32B_W8A16 = {
    "top": {"model_type": "qwen3_vl", "tie_word_embeddings": False},
    "quant_config": {"method": W8A16_METHOD, "mode": "per_channel_symmetric", "qaxis": 0, "skip_modules": ["lm_head"],
                     "quantized_lm_head": False, "quantized_embed_tokens": False, "lm_head_untied": False,
                     "embed_tokens_untied": False},
    "text_config": {"model_type": "qwen3_vl_text", "hidden_size": 5120, "intermediate_size": 25600,
                    "num_hidden_layers": 64, "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128,
                    "vocab_size": 151936, "hidden_act": "silu", "rms_norm_eps": 1e-6},
    "vision_config": {"model_type": "qwen3_vl", "hidden_size": 1152, "intermediate_size": 4304, "depth": 27,
                      "num_heads": 16, "patch_size": 16, "temporal_patch_size": 2, "spatial_merge_size": 2,
                      "deepstack_visual_indexes": [8, 16, 24], "out_hidden_size": 5120,
                      "hidden_act": "gelu_pytorch_tanh"},
}


def is_qwen3_vl_32b_w8a16_config(config) -> bool:
    """True only for the exact profile above; anything missing, extra-quantised or differently sized is False."""
    read = (lambda o, k: o.get(k)) if isinstance(config, dict) else (lambda o, k: getattr(o, k, None))

    def matches(obj, want: dict) -> bool:
        if obj is None:
            return False
        get = (lambda k: obj.get(k)) if isinstance(obj, dict) else (lambda k: getattr(obj, k, None))
        for key, value in want.items():
            got = get(key)
            if isinstance(value, float):
                if not isinstance(got, (int, float)) or abs(float(got) - value) > 1e-12:
                    return False
            elif isinstance(value, list):
                if got is None or list(got) != value:
                    return False
            elif got != value or isinstance(got, bool) != isinstance(value, bool):
                return False
        return True

    arch = read(config, "architectures")
    return (arch is not None and tuple(arch) == ("Qwen3VLForConditionalGeneration",)
            and matches(config, QWEN3_VL_32B_W8A16["top"])
            and read(config, "quant_config") == QWEN3_VL_32B_W8A16["quant_config"]
            and matches(read(config, "text_config"), QWEN3_VL_32B_W8A16["text_config"])
            and matches(read(config, "vision_config"), QWEN3_VL_32B_W8A16["vision_config"]))


def w4a16_tensor_getter(ckpt_dir: str, config) -> Callable[[str], torch.Tensor]:
    """``get(name)`` over a packed W4A16 checkpoint (``quant/convert_qwen3_w4a16.py``): a packed projection
    (``uint8 [out, in/2]`` with group-wise fp16 scales) is dequantised to fp16 when it is read, so the 16-bit kernels run
    it; there is no 4-bit device GEMM.  Every other tensor is returned as stored; scale tensors are not listed."""
    from ..api._loading import checkpoint_tensor_getter
    from .int4_pgrp_pack import dequantize_int4_pgrp
    qc = getattr(config, "quant_config", None) or (config.get("quant_config") if isinstance(config, dict) else {})
    group = int(qc.get("group_size", 32))
    base = checkpoint_tensor_getter(ckpt_dir)
    scale_of = lambda n: n[:-len(".weight")] + ".weight_scale"

    def get(name: str) -> torch.Tensor:
        t = base(name)
        if t.dtype == torch.uint8 and name.endswith(".weight") and scale_of(name) in base.names:
            return dequantize_int4_pgrp(t, base(scale_of(name)), group)
        return t

    get.names = frozenset(n for n in base.names if not n.endswith(".weight_scale"))  # type: ignore[attr-defined]
    return get


def _shards(ckpt: Path) -> List[Path]:
    idx = ckpt / "model.safetensors.index.json"
    if idx.is_file():
        wm = json.loads(idx.read_text())["weight_map"]
        return [ckpt / s for s in sorted(set(wm.values()))]
    single = ckpt / "model.safetensors"
    if single.is_file():
        return [single]
    raise FileNotFoundError(f"no safetensors checkpoint in {ckpt}")


def w8a16_tensor_getter(ckpt_dir: str, config=None) -> Callable[[str], torch.Tensor]:
    """``get(name)`` over a W8A16 checkpoint; ``get.scale(name)`` returns the fp16 per-channel scale
    of an int8 tensor (or ``None``), ``get.names`` the tensor names present."""
    from ..api._loading import checkpoint_tensor_getter
    base = checkpoint_tensor_getter(ckpt_dir)
    names = base.names

    def get(name: str) -> torch.Tensor:
        if name == LM_HEAD and name not in names:
            return base(EMBED)
        t = base(name)
        if name.endswith(PROJECTION_SUFFIXES) and t.dtype != torch.int8 and scale_name(name) in names:
            raise TypeError(f"W8A16 projection {name!r} must be int8, got {t.dtype}")
        return t

    def scale(name: str):
        if name == LM_HEAD and name not in names:
            name = EMBED
        sn = scale_name(name)
        return base(sn).to(torch.float16) if sn in names else None

    get.scale = scale      # type: ignore[attr-defined]
    get.names = names      # type: ignore[attr-defined]
    return get


def _set_tensor(model: nn.Module, name: str, tensor: torch.Tensor) -> None:
    """Install a checkpoint tensor over the skeleton's parameter or buffer of the same name; the shapes must agree
    (a mis-sized checkpoint is an error here, not wrong numbers later)."""
    mod_name, _, leaf = name.rpartition(".")
    mod = model.get_submodule(mod_name) if mod_name else model
    if leaf in mod._parameters:
        old = mod._parameters[leaf]
    elif leaf in mod._buffers:
        old = mod._buffers[leaf]
    else:
        raise KeyError(f"checkpoint tensor {name!r} has no destination in the model")
    if old is not None and tuple(old.shape) != tuple(tensor.shape):
        raise ValueError(f"checkpoint tensor {name!r} has shape {tuple(tensor.shape)}, the model expects {tuple(old.shape)}")
    if leaf in mod._parameters:
        mod._parameters[leaf] = nn.Parameter(tensor, requires_grad=False)
    else:
        mod._buffers[leaf] = tensor


def _skipped(name: str, skip_modules) -> bool:
    """True when ``name`` belongs to a module the converter was told to leave in 16 bits."""
    return any(s and (name == s + ".weight" or name.startswith(s + ".") or ("." + s + ".") in ("." + name))
               for s in (skip_modules or ()))


def _rope_init(mod):
    """The function a Hugging Face rotary-embedding module derives its ``inv_freq`` with (by rope type)."""
    fn = getattr(mod, "rope_init_fn", None)
    if fn is not None:
        return fn
    rope_type = getattr(mod, "rope_type", "default")
    if rope_type != "default":
        from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
        return ROPE_INIT_FUNCTIONS[rope_type]
    return mod.compute_default_rope_parameters


def load_w8a16_model(config, ckpt_dir: str, *, dtype: torch.dtype = torch.float16, **_ignored) -> nn.Module:
    """CPU model with int8 projection Parameters and ``weight_scale`` buffers; every other tensor in
    ``dtype``.  Fails on partial loads (a projection without its scale, or left on ``meta``)."""
    from safetensors.torch import load_file
    from transformers import AutoModelForCausalLM
    ckpt = Path(ckpt_dir)
    qc = getattr(config, "quant_config", None) or {}
    skip = tuple(qc.get("skip_modules") or ())
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(config)
    seen: set = set()
    for shard in _shards(ckpt):
        for name, t in load_file(str(shard)).items():
            if name.endswith(".weight_scale"):
                owner_name = name[:-len(".weight_scale")]
                owner = model.get_submodule(owner_name)
                rows = getattr(owner, "weight").shape[0]
                if t.dtype != torch.float16 or t.numel() != rows:
                    raise ValueError(f"{name!r} must be fp16 with one entry per output row ({rows}), got {t.dtype} "
                                     f"x {t.numel()}")
                owner.register_buffer("weight_scale", t)
                seen.add(name)
                continue
            if t.dtype == torch.int8:
                if not (name.endswith(PROJECTION_SUFFIXES) or name in (LM_HEAD, EMBED)):
                    raise TypeError(f"unexpected int8 tensor {name!r} in a W8A16 checkpoint")
                _set_tensor(model, name, t)
            else:
                if name.endswith(PROJECTION_SUFFIXES) and t.is_floating_point() and not _skipped(name, skip):
                    raise TypeError(f"W8A16 projection {name!r} must be int8, got {t.dtype}")
                _set_tensor(model, name, t.to(dtype) if t.is_floating_point() else t)
            seen.add(name)
    if getattr(config, "tie_word_embeddings", False) and LM_HEAD not in seen:
        model.lm_head.weight = model.model.embed_tokens.weight
    for n, p in model.named_parameters():
        if p.is_meta:
            raise RuntimeError(f"W8A16 checkpoint left {n!r} unloaded")
        if p.dtype == torch.int8 and scale_name(n) not in seen:
            raise RuntimeError(f"W8A16 tensor {n!r} has no {scale_name(n)!r}")
    # Buffers the checkpoint does not carry were created on meta and need real storage.  Only the rotary
    # frequencies can be rebuilt from the configuration (with the attention scaling of non-default rope types);
    # anything else left on meta is an error rather than a zero fill.
    for mname, mod in model.named_modules():
        for bn, b in list(mod._buffers.items()):
            if b is None or not b.is_meta:
                continue
            if bn in ("inv_freq", "original_inv_freq") and hasattr(mod, "config"):
                inv, scaling = _rope_init(mod)(mod.config, torch.device("cpu"))
                mod._buffers[bn] = inv.clone()
                if hasattr(mod, "attention_scaling"):
                    mod.attention_scaling = scaling
            else:
                raise KeyError(f"buffer {mname + '.' if mname else ''}{bn} is neither in the checkpoint nor derivable "
                               "from the configuration")
    model._rpu_w8a16 = True
    return model.eval()


__all__ = ["is_w8a16_config", "load_w8a16_model", "w8a16_tensor_getter", "W8A16_METHOD"]
