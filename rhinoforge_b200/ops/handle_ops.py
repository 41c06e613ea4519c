"""Handle-family operators of ``torch.ops.rpu``: ``<family>_create / _set_weights[_w8a16] / _forward / _destroy``.

The reference exposes every fused model runtime as an integer handle behind dispatcher ops
(``src/core/rpu_dispatch_registrations.inc:29-139,853-1019``).  Here the runtimes are Python objects over the
native stack executor; this module gives them the same by-name surface: a handle is an integer key of a
process-wide table, ``*_create`` takes the model configuration as a JSON string, ``*_set_weights`` takes
parallel lists of checkpoint names and tensors and builds the device runtime, ``*_forward`` runs it and
``*_destroy`` releases it.  Differences that follow from the B200 design: KV caches are the engine's paged
pool (the ``k_caches`` / ``v_caches`` lists of ``causal_decoder_forward`` are accepted for signature parity
and not read), and the decoder returns last-row logits of each sequence (the reference's fused-lm-head mode).

Families: ``causal_decoder`` and ``qwen3_5`` (``runtime.engine.DecoderEngine``), ``qwen3vl_vision`` /
``qwen3_5_vision`` (``models.vision.Qwen3VLVisionEncoder``), ``qwen25vl_vision``, ``siglip``, ``hyvit2`` (optional
projector passed as ``rpu_projector.weight`` / ``rpu_projector.bias``), ``dinov3_vision``,
and the Pi0.5 set ``pi05`` / ``gemma`` / ``adarms`` / ``pi05_denoise_step`` (+ ``pi05_denoise_loop_forward``), which
share one ``models.pi05.Pi05Engine`` per handle: ``gemma_forward`` is the prefix pass, ``adarms_forward`` /
``pi05_denoise_step_forward`` / ``pi05_denoise_loop_forward`` integrate the action expert over the stored prefix.
"""
from __future__ import annotations

import json
import threading
from types import SimpleNamespace
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..runtime.errors import RPUBackendError, RPUConfigError

_LOCK = threading.Lock()
_TABLE: Dict[int, "_Entry"] = {}
_NEXT = [1]


class _Entry:
    def __init__(self, family: str, config: dict):
        self.family, self.config = family, config
        self.runtime: Any = None
        self.state: Dict[str, Any] = {}


def _create(family: str, config_json: str) -> int:
    try:
        cfg = json.loads(config_json) if config_json else {}
    except json.JSONDecodeError as e:
        raise RPUConfigError(f"{family}_create: configuration is not valid JSON: {e}") from None
    if not isinstance(cfg, dict):
        raise RPUConfigError(f"{family}_create: configuration must be a JSON object")
    with _LOCK:
        h = _NEXT[0]
        _NEXT[0] += 1
        _TABLE[h] = _Entry(family, cfg)
    return h


def _entry(handle: int, families: Sequence[str]) -> _Entry:
    e = _TABLE.get(int(handle))
    if e is None:
        raise RPUBackendError(f"unknown or destroyed handle {handle}")
    if e.family not in families:
        raise RPUBackendError(f"handle {handle} belongs to family {e.family!r}, not {'/'.join(families)}")
    return e


def _destroy(handle: int, families: Sequence[str]) -> None:
    e = _entry(handle, families)
    with _LOCK:
        _TABLE.pop(int(handle), None)
    if e.runtime is not None and hasattr(e.runtime, "close"):
        e.runtime.close()


def live_handles() -> Dict[int, str]:
    """Handle -> family of every live handle (debug surface)."""
    return {h: e.family for h, e in _TABLE.items()}


def _sd(names: Sequence[str], tensors: Sequence[torch.Tensor]) -> Dict[str, torch.Tensor]:
    if len(names) != len(tensors):
        raise RPUBackendError(f"set_weights: {len(names)} names for {len(tensors)} tensors")
    return dict(zip(names, tensors))


def _runtime(e: _Entry):
    if e.runtime is None:
        raise RPUBackendError(f"{e.family} handle has no weights yet: call {e.family}_set_weights first")
    return e.runtime


def _dtype_of(cfg: dict):
    return {"float16": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}[
        str(cfg.get("torch_dtype", cfg.get("dtype", "float16"))).replace("torch.", "")]


# ------------------------------------------------------------------------------------------ decoders
_DECODERS = ("causal_decoder", "qwen3_5")


def _decoder_set_weights(handle: int, names: List[str], tensors: List[torch.Tensor], quant: Optional[str]) -> None:
    from ..models.decoder import DecoderConfig
    from ..runtime.engine import DecoderEngine
    e = _entry(handle, _DECODERS)
    if e.runtime is not None:
        e.runtime.close()
    sd = _sd(names, tensors)
    hf = SimpleNamespace(**e.config)
    cfg = DecoderConfig.from_hf(hf)

    def get(name: str) -> torch.Tensor:
        if name not in sd and name.startswith("model.") and name[6:] in sd:
            return sd[name[6:]]
        return sd[name]
    e.runtime = DecoderEngine(cfg, get, dtype=_dtype_of(e.config), max_batch=int(e.config.get("rpu_max_batch", 1)),
                              max_seq_len=int(e.config.get("rpu_max_seq_len", 2048)),
                              max_prefill_tokens=int(e.config.get("rpu_max_prefill_tokens", 8192)), quant=quant)


def _decoder_forward(handle: int, hidden_states: torch.Tensor, k_caches: List[torch.Tensor], v_caches: List[torch.Tensor],
                     attention_mask: Optional[torch.Tensor], position: int, is_causal: bool,
                     position_ids: Optional[torch.Tensor], deepstack_dense_visual_embeds: Optional[List[torch.Tensor]],
                     rope_cos_il: Optional[torch.Tensor], rope_sin_il: Optional[torch.Tensor], cos_sin_offset: int = -1,
                     batch_slot: int = 0, allow_batch_decode: bool = False) -> torch.Tensor:
    """``hidden_states [B, S, hidden]`` (input embeddings) appended at ``position`` -> last-row logits ``[B, vocab]``.

    ``position == 0`` starts the sequences from empty; any other value must equal the tokens already cached.
    ``position_ids`` ``[3, B, S]`` selects M-RoPE.  Masks other than causal are not part of this family."""
    eng = _runtime(_entry(handle, _DECODERS))
    if not is_causal or attention_mask is not None:
        raise RPUBackendError("causal_decoder_forward runs causal attention over the paged cache; explicit masks "
                              "belong to the prefix-LM runtimes")
    if hidden_states.dim() == 2:
        hidden_states = hidden_states[None]
    B = hidden_states.shape[0]
    if position == 0:
        eng.reset()
    elif any(eng.cache.lengths[s] != position for s in range(B)):
        raise RPUBackendError(f"position {position} does not match the cached lengths "
                              f"{[eng.cache.lengths[s] for s in range(B)]}")
    S = hidden_states.shape[1]
    tokens = [torch.zeros(S, dtype=torch.int32) for _ in range(B)]
    embeds = [hidden_states[b].to(eng.device, eng.dtype).contiguous() for b in range(B)]
    pos3 = None
    if position_ids is not None and position_ids.dim() == 3:
        pos3 = [position_ids[:, b].to(torch.int32) for b in range(B)]
    _, logits = eng.extend(tokens, return_logits=True, inputs_embeds=embeds, positions3=pos3)
    return logits


# ------------------------------------------------------------------------------------------ vision towers
def _vision_set_weights(family: str, handle: int, names: List[str], tensors: List[torch.Tensor]) -> None:
    e = _entry(handle, (family,))
    if e.runtime is not None:
        e.runtime.close()
    sd, cfg, dt = _sd(names, tensors), e.config, _dtype_of(e.config)
    if family in ("qwen3vl_vision", "qwen3_5_vision"):
        from ..models.vision import Qwen3VLVisionConfig, Qwen3VLVisionEncoder
        c = Qwen3VLVisionConfig.from_hf(cfg)
        if family == "qwen3_5_vision":
            c.deepstack_visual_indexes = ()
        e.runtime = Qwen3VLVisionEncoder(c, sd, dtype=dt, max_patches=int(cfg.get("rpu_max_patches", 4096)))
    elif family == "qwen25vl_vision":
        from ..models.qwen25_vl_vision import Qwen25VLVisionConfig, Qwen25VLVisionEncoder
        e.runtime = Qwen25VLVisionEncoder(Qwen25VLVisionConfig.from_hf(cfg), sd, dtype=dt,
                                          max_patches=int(cfg.get("rpu_max_patches", 4096)))
    elif family == "siglip":
        from ..models.vision import SiglipConfig, SiglipVisionEncoder
        e.runtime = SiglipVisionEncoder(SiglipConfig.from_hf(cfg), sd, prefix=str(cfg.get("rpu_prefix", "vision_model.")),
                                        dtype=dt, max_images=int(cfg.get("rpu_max_images", 8)))
    elif family == "hyvit2":
        from ..models.vision import HYViT2Encoder, SiglipConfig
        proj = None
        if "rpu_projector.weight" in sd:
            proj = (sd.pop("rpu_projector.weight"), sd.pop("rpu_projector.bias"))
        e.runtime = HYViT2Encoder(SiglipConfig.from_hf(cfg), sd, prefix=str(cfg.get("rpu_prefix", "")), dtype=dt,
                                  max_images=int(cfg.get("rpu_max_images", 1)), projector=proj)
    elif family == "dinov3_vision":
        from ..models.vision import DINOv3Config, DINOv3Encoder
        e.runtime = DINOv3Encoder(DINOv3Config.from_hf(cfg), sd, dtype=dt)
    else:  # pragma: no cover
        raise RPUBackendError(f"unknown vision family {family}")


def _grid_vision_forward(family: str, handle: int, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> List[torch.Tensor]:
    out = _runtime(_entry(handle, (family,)))(pixel_values, grid_thw)
    if isinstance(out, tuple):
        emb, deep = out
        return [emb] + list(deep)
    return [out]


def _image_vision_forward(family: str, handle: int, pixel_values: torch.Tensor) -> List[torch.Tensor]:
    out = _runtime(_entry(handle, (family,)))(pixel_values)
    return list(out) if isinstance(out, tuple) else [out]


# ------------------------------------------------------------------------------------------ Pi0.5
_PI05 = ("pi05", "gemma", "adarms", "pi05_denoise_step")


def _pi05_config(cfg: dict):
    from ..models.pi05 import GemmaGeometry, Pi05Config
    from ..models.vision import SiglipConfig
    kw = {k: v for k, v in cfg.items() if k in ("vocab_size", "action_dim", "horizon", "min_period", "max_period",
                                                "max_lang_tokens", "num_views")}
    for part, cls in (("vlm", GemmaGeometry), ("expert", GemmaGeometry), ("vision", SiglipConfig)):
        if part in cfg:
            kw[part] = cls(**cfg[part])
    return Pi05Config(**kw)


def _pi05_set_weights(handle: int, names: List[str], tensors: List[torch.Tensor]) -> None:
    from ..models.pi05 import Pi05Engine
    e = _entry(handle, _PI05)
    if e.runtime is not None:
        e.runtime.close()
    e.runtime = Pi05Engine(_pi05_config(e.config), _sd(names, tensors), dtype=_dtype_of(e.config),
                           max_batch=int(e.config.get("rpu_max_batch", 1)))


def _pi05_forward(handle: int, images: torch.Tensor, image_mask: torch.Tensor, tokens: torch.Tensor, token_mask: torch.Tensor,
                  noise: torch.Tensor, num_steps: int = 10) -> torch.Tensor:
    return _runtime(_entry(handle, _PI05)).predict(images, image_mask, tokens, token_mask, noise, num_steps)


def _gemma_forward(handle: int, images: torch.Tensor, image_mask: torch.Tensor, tokens: torch.Tensor,
                   token_mask: torch.Tensor) -> torch.Tensor:
    """Prefix pass (vision + language through the Gemma backbone into the prefix KV): returns the prefix lengths."""
    e = _entry(handle, _PI05)
    lens = _runtime(e).prefill(images, image_mask, tokens, token_mask)
    e.state["prefix_lens"] = [int(v) for v in lens]
    return torch.tensor(e.state["prefix_lens"], dtype=torch.int32)


def _denoise_forward(handle: int, prefix_lens: Optional[torch.Tensor], noise: torch.Tensor, num_steps: int = 10) -> torch.Tensor:
    e = _entry(handle, _PI05)
    lens = [int(v) for v in prefix_lens.tolist()] if prefix_lens is not None else e.state.get("prefix_lens")
    if lens is None:
        raise RPUBackendError("no prefix is stored on this handle: run gemma_forward first or pass prefix_lens")
    return _runtime(e).denoise(lens, noise, num_steps)


# ------------------------------------------------------------------------------------------ registration
# ------------------------------------------------------------------------------------------ action heads
# Flow-matching / diffusion heads: the handle's configuration is the dataclass of the engine as a JSON object
# (``{}`` = the published profile); ``set_weights`` takes the checkpoint's own tensor names.
_HEADS = ("navdp", "gr00t", "internvla_nextdit", "rhino_vla", "qwenpi05", "gemma4")


def _head_cfg(cls, cfg: dict):
    fields = getattr(cls, "__dataclass_fields__", {})
    return cls(**{k: v for k, v in cfg.items() if k in fields})


def _head_set_weights(family: str, handle: int, names: List[str], tensors: List[torch.Tensor]) -> None:
    e = _entry(handle, (family,))
    if e.runtime is not None:
        e.runtime.close()
    sd, cfg, dtype = _sd(names, tensors), e.config, _dtype_of(e.config)
    if family == "navdp":
        from ..models.navdp import NavdpConfig, NavdpEngine
        e.runtime = NavdpEngine(_head_cfg(NavdpConfig, cfg), sd, max_samples=int(cfg.get("rpu_max_samples", 4)), dtype=dtype)
    elif family == "gr00t":
        from ..models.gr00t import Gr00tConfig, Gr00tEngine
        e.runtime = Gr00tEngine(_head_cfg(Gr00tConfig, cfg), sd.__getitem__, embodiment=int(cfg.get("rpu_embodiment", 0)),
                                max_vl=int(cfg.get("rpu_max_vl", 512)), dtype=dtype)
    elif family == "internvla_nextdit":
        from ..models.nextdit import NextDiTConfig, NextDiTEngine
        e.runtime = NextDiTEngine(_head_cfg(NextDiTConfig, cfg), sd, dtype=dtype)
    elif family == "rhino_vla":
        from ..models.rhinovla import RhinoVLAConfig, RhinoVLAEngine
        e.runtime = RhinoVLAEngine(_head_cfg(RhinoVLAConfig, cfg), sd, max_prefix=int(cfg.get("rpu_max_prefix", 1024)), dtype=dtype)
    elif family == "qwenpi05":
        from ..models.qwenpi05 import QwenPI05Config, QwenPI05Engine
        e.runtime = QwenPI05Engine(_head_cfg(QwenPI05Config, cfg), sd, max_prefix=int(cfg.get("rpu_max_prefix", 1024)), dtype=dtype)
    elif family == "gemma4":
        from ..models.gemma4 import Gemma4Engine
        text = {k: v for k, v in cfg.items() if not k.startswith("rpu_")}
        e.runtime = Gemma4Engine(text, sd.__getitem__, prefix=str(cfg.get("rpu_weight_prefix", "model.")),
                                 max_seq_len=int(cfg.get("rpu_max_seq_len", 2048)), max_batch=int(cfg.get("rpu_max_batch", 1)),
                                 max_tokens=int(cfg.get("rpu_max_prefill_tokens", cfg.get("rpu_max_seq_len", 2048))), dtype=dtype)


def _navdp_forward(handle: int, goal_embed: torch.Tensor, rgbd_embed: torch.Tensor, init_noise: torch.Tensor,
                   step_noise: torch.Tensor) -> torch.Tensor:
    return _runtime(_entry(handle, ("navdp",))).predict_action(goal_embed, rgbd_embed, init_noise, step_noise)


def _gr00t_vl_forward(handle: int, hidden: torch.Tensor) -> torch.Tensor:
    return _runtime(_entry(handle, ("gr00t",))).vl_encode(hidden).clone()


def _gr00t_denoise_forward(handle: int, noise: torch.Tensor, state: torch.Tensor, vl_embeds: torch.Tensor, image_mask: torch.Tensor,
                           valid_mask: Optional[torch.Tensor]) -> torch.Tensor:
    return _runtime(_entry(handle, ("gr00t",))).denoise(vl_embeds, state, noise, image_mask, valid_mask)


def _nextdit_forward(handle: int, actions: torch.Tensor, timesteps: torch.Tensor, euler_steps: torch.Tensor,
                     condition: torch.Tensor) -> torch.Tensor:
    return _runtime(_entry(handle, ("internvla_nextdit",))).denoise_actions(actions, timesteps, euler_steps, condition)


def _expert_set_prefix(families, handle: int, keys: List[torch.Tensor], values: List[torch.Tensor], prefix_valid: Optional[torch.Tensor]) -> int:
    if len(keys) != len(values):
        raise RPUBackendError(f"set_prefix: {len(keys)} key tensors for {len(values)} value tensors")
    return int(_runtime(_entry(handle, families)).set_prefix(list(zip(keys, values)), prefix_valid))


def _rhino_forward(handle: int, state: torch.Tensor, noise: torch.Tensor, state_mask: Optional[torch.Tensor],
                   action_mask: Optional[torch.Tensor], cond_all: Optional[torch.Tensor]) -> torch.Tensor:
    rt = _runtime(_entry(handle, ("rhino_vla",)))
    return rt.predict(state, noise, state_mask=state_mask, action_mask=action_mask, cond_all=cond_all).clone()


def _qwenpi05_forward(handle: int, state: Optional[torch.Tensor], noise: torch.Tensor, num_steps: int = 10) -> torch.Tensor:
    return _runtime(_entry(handle, ("qwenpi05",))).predict(state, noise, num_steps).clone()


def _gemma4_forward(handle: int, input_ids: torch.Tensor, reset: bool = True) -> torch.Tensor:
    """``input_ids [B, L]`` appended to sequences ``0 .. B-1`` (from empty when ``reset``) -> last-row logits ``[B, vocab]`` fp32."""
    rt = _runtime(_entry(handle, ("gemma4",)))
    rows = [input_ids[b] for b in range(input_ids.shape[0])] if input_ids.dim() == 2 else [input_ids]
    if reset:
        rt.reset()
    return rt.extend(rows)


def register(lib: "torch.library.Library") -> None:
    """Define and implement the handle-family schemas on ``lib`` (the ``rpu`` namespace)."""
    def op(schema: str, fn) -> None:
        lib.define(schema)
        lib.impl(schema.split("(")[0], fn, "CompositeExplicitAutograd")

    def family(name: str, families: Sequence[str], set_weights, forward_schema: str, forward, w8a16=None) -> None:
        op(f"{name}_create(str config_json) -> int", lambda config_json, _n=name: _create(_n, config_json))
        op(f"{name}_destroy(int handle) -> ()", lambda handle, _f=tuple(families): _destroy(handle, _f))
        op(f"{name}_set_weights(int handle, str[] names, Tensor[] tensors) -> ()", set_weights)
        if w8a16 is not None:
            op(f"{name}_set_weights_w8a16(int handle, str[] names, Tensor[] tensors) -> ()", w8a16)
        op(f"{name}_forward{forward_schema}", forward)

    dec_schema = ("(int handle, Tensor hidden_states, Tensor[] k_caches, Tensor[] v_caches, Tensor? attention_mask, "
                  "int position, bool is_causal, Tensor? position_ids, Tensor[]? deepstack_dense_visual_embeds, "
                  "Tensor? rope_cos_il, Tensor? rope_sin_il, int cos_sin_offset=-1, int batch_slot=0, "
                  "bool allow_batch_decode=False) -> Tensor")
    for name in _DECODERS:
        family(name, _DECODERS, lambda handle, names, tensors: _decoder_set_weights(handle, names, tensors, None),
               dec_schema, _decoder_forward,
               w8a16=lambda handle, names, tensors: _decoder_set_weights(handle, names, tensors, "w8a16"))
    for name in ("qwen3vl_vision", "qwen3_5_vision", "qwen25vl_vision"):
        family(name, (name,), lambda handle, names, tensors, _n=name: _vision_set_weights(_n, handle, names, tensors),
               "(int handle, Tensor pixel_values, Tensor grid_thw) -> Tensor[]",
               lambda handle, pixel_values, grid_thw, _n=name: _grid_vision_forward(_n, handle, pixel_values, grid_thw))
    for name in ("siglip", "hyvit2", "dinov3_vision"):
        family(name, (name,), lambda handle, names, tensors, _n=name: _vision_set_weights(_n, handle, names, tensors),
               "(int handle, Tensor pixel_values) -> Tensor[]",
               lambda handle, pixel_values, _n=name: _image_vision_forward(_n, handle, pixel_values))
    family("pi05", _PI05, _pi05_set_weights,
           "(int handle, Tensor images, Tensor image_mask, Tensor tokens, Tensor token_mask, Tensor noise, int num_steps=10) -> Tensor",
           _pi05_forward)
    family("gemma", _PI05, _pi05_set_weights,
           "(int handle, Tensor images, Tensor image_mask, Tensor tokens, Tensor token_mask) -> Tensor", _gemma_forward)
    for name in ("adarms", "pi05_denoise_step"):
        family(name, _PI05, _pi05_set_weights, "(int handle, Tensor? prefix_lens, Tensor noise, int num_steps=10) -> Tensor",
               _denoise_forward)
    op("pi05_denoise_loop_forward(int handle, Tensor? prefix_lens, Tensor noise, int num_steps=10) -> Tensor", _denoise_forward)

    def head(name: str, forward_schema: str, forward) -> None:
        family(name, (name,), lambda handle, names, tensors, _n=name: _head_set_weights(_n, handle, names, tensors),
               forward_schema, forward)

    head("navdp", "(int handle, Tensor goal_embed, Tensor rgbd_embed, Tensor init_noise, Tensor step_noise) -> Tensor", _navdp_forward)
    head("gr00t", "(int handle, Tensor noise, Tensor state, Tensor vl_embeds, Tensor image_mask, Tensor? valid_mask) -> Tensor",
         _gr00t_denoise_forward)
    op("gr00t_vl_encoder_forward(int handle, Tensor hidden) -> Tensor", _gr00t_vl_forward)
    op("gr00t_denoise_unroll_forward(int handle, Tensor noise, Tensor state, Tensor vl_embeds, Tensor image_mask, Tensor? valid_mask) -> Tensor",
       _gr00t_denoise_forward)
    head("internvla_nextdit", "(int handle, Tensor actions, Tensor timesteps, Tensor euler_steps, Tensor condition) -> Tensor",
         _nextdit_forward)
    head("rhino_vla", "(int handle, Tensor state, Tensor noise, Tensor? state_mask, Tensor? action_mask, Tensor? cond_all) -> Tensor",
         _rhino_forward)
    head("qwenpi05", "(int handle, Tensor? state, Tensor noise, int num_steps=10) -> Tensor", _qwenpi05_forward)
    for name in ("rhino_vla", "qwenpi05"):
        op(f"{name}_set_prefix(int handle, Tensor[] keys, Tensor[] values, Tensor? prefix_valid) -> int",
           lambda handle, keys, values, prefix_valid, _f=(name,): _expert_set_prefix(_f, handle, keys, values, prefix_valid))
    head("gemma4", "(int handle, Tensor input_ids, bool reset=True) -> Tensor", _gemma4_forward)


FAMILIES = _DECODERS + ("qwen3vl_vision", "qwen3_5_vision", "qwen25vl_vision", "siglip", "hyvit2", "dinov3_vision") + _PI05 + _HEADS

__all__ = ["register", "live_handles", "FAMILIES"]
