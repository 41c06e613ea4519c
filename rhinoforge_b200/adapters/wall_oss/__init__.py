"""Wall-OSS adapter: checkpoint configuration -> :class:`rhinoforge_b200.models.wall_oss.WallOssEngine`, plus the host
glue of one inference (prompt text, proprioception string, normaliser files).

``config.json`` is a flat Qwen2.5-VL configuration with two additions: ``experts`` (a list of two
``{hidden_size, intermediate_size}`` blocks: the prompt decoder and the action decoder) and ``action_hidden_size``.
The attention geometry (heads, KV heads, head size, layer count) is shared by both experts.  All rejections are decided
from the configuration before a weight is read.

Reference: ``python/rpu_backend/adapters/wall_oss/runtime.py:208-300,1078-1090,1465-1810`` (prompt, state string,
build), ``adapters/wall_oss/llm.py:950-1000`` and ``adapters/wall_oss/action.py:1046-1060`` (configuration keys).
"""
from __future__ import annotations

import os
from typing import Callable, Mapping, Optional, Sequence

import numpy as np
import torch

from ...api.errors import RPUConfigError, UnsupportedModelError
from ...models.decoder import DecoderConfig
from ...models.qwen25_vl_vision import Qwen25VLVisionConfig
from ...models.wall_oss import PRE_P, WallOssConfig, wall_oss_action_shapes, wall_oss_expert_shapes

IMAGE_PAD_ID = 151655

# raw camera key -> the prose name the prompt uses
CAMERA_PROSE = {
    "face_view": "front view", "left_wrist_view": "left wrist view", "right_wrist_view": "right wrist view",
    "move1_view": "move view", "move2_view": "move view", "wall_view": "wall view", "top_view": "top view",
    "side_view": "side view", "global_view": "global view",
}
PROMPT_STYLES = ("default", "short", "generic", "multisuite")


def _expert(config: Mapping, i: int) -> Mapping:
    ex = config.get("experts")
    if not isinstance(ex, (list, tuple)) or len(ex) < 2 or not all(isinstance(e, Mapping) for e in ex[:2]):
        raise UnsupportedModelError("Wall-OSS config.json must carry `experts`: two {hidden_size, intermediate_size} blocks")
    return ex[i]


def text_config(config: Mapping) -> DecoderConfig:
    """Decoder configuration of expert 0 (the Qwen2.5 prompt decoder)."""
    rs = config.get("rope_scaling") or {}
    if not rs.get("mrope_section"):
        raise UnsupportedModelError("Wall-OSS config.json carries no rope_scaling.mrope_section")
    e0 = _expert(config, 0)
    heads = int(config["num_attention_heads"])
    H = int(e0.get("hidden_size", config["hidden_size"]))
    return DecoderConfig(
        name="wall-oss-expert0", vocab_size=int(config["vocab_size"]), hidden_size=H,
        intermediate_size=int(e0.get("intermediate_size", config.get("intermediate_size", 0))),
        num_layers=int(config["num_hidden_layers"]), num_heads=heads,
        num_kv_heads=int(config.get("num_key_value_heads", heads)),
        head_dim=int(config.get("head_dim") or int(config["hidden_size"]) // heads), rms_eps=float(config.get("rms_norm_eps", 1e-6)),
        rope_theta=float(config.get("rope_theta", 1e6)), tie_embeddings=bool(config.get("tie_word_embeddings", False)),
        qk_norm=False, attention_bias=True, max_position=int(config.get("max_position_embeddings", 32768)),
        mrope_section=tuple(int(v) for v in rs["mrope_section"]), mrope_interleaved=False, model_type="qwen2_5_vl")


def action_config(config: Mapping, *, action_dim: int, horizon: int = 32, num_steps: int = 10, causal_actions: bool = True,
                  flow_time_scale: float = 1.0) -> WallOssConfig:
    t = text_config(config)
    e1 = _expert(config, 1)
    cfg = WallOssConfig(hidden=int(e1["hidden_size"]), inter=int(e1["intermediate_size"]), layers=t.num_layers, heads=t.num_heads,
                        kv_heads=t.num_kv_heads, head_dim=t.head_dim, eps=t.rms_eps, rope_theta=t.rope_theta,
                        action_dim=int(action_dim), horizon=int(horizon), num_steps=int(num_steps),
                        causal_actions=bool(causal_actions), flow_time_scale=float(flow_time_scale))
    ah = int(config.get("action_hidden_size", cfg.hidden))
    if ah != cfg.hidden:
        raise UnsupportedModelError(f"action_hidden_size {ah} differs from the action decoder's width {cfg.hidden}")
    preflight(cfg)
    return cfg


def preflight(cfg: WallOssConfig) -> None:
    bad = []
    if cfg.head_dim not in (64, 128, 256):
        bad.append(f"head_dim {cfg.head_dim} (64 / 128 / 256)")
    if cfg.hidden % 8 or cfg.inter % 8:
        bad.append("widths that are not multiples of 8")
    if cfg.heads % cfg.kv_heads:
        bad.append(f"{cfg.heads} query heads over {cfg.kv_heads} kv heads")
    if cfg.num_steps < 1 or cfg.horizon < 1 or cfg.action_dim < 1:
        bad.append("an empty denoise schedule or action chunk")
    if bad:
        raise UnsupportedModelError("Wall-OSS configuration is outside what this framework runs: " + "; ".join(bad))


def build_engine(config: Mapping, get_weight: Callable[[str], torch.Tensor], *, horizon: int = 32, num_steps: int = 10,
                 max_seq_len: int = 2048, max_patches: int = 4096, causal_actions: bool = True, flow_time_scale: float = 1.0,
                 device="cuda", dtype=torch.float16):
    from ...models.wall_oss import WallOssEngine
    names = getattr(get_weight, "names", None)
    back = get_weight(PRE_P + "action_proj_back.weight")
    cfg = action_config(config, action_dim=int(back.shape[0]), horizon=horizon, num_steps=num_steps,
                        causal_actions=causal_actions, flow_time_scale=flow_time_scale)
    if names is not None:
        want = [n for n, _, _ in list(wall_oss_expert_shapes(cfg)) + list(wall_oss_action_shapes(cfg))]
        missing = [n for n in want if n not in names]
        if missing:
            raise UnsupportedModelError(f"checkpoint lacks {len(missing)} action-decoder tensors, first: {missing[0]!r}")
    if max_seq_len <= cfg.horizon:
        raise ValueError(f"max_seq_len {max_seq_len} leaves no room for a prompt before {cfg.horizon} action rows")
    vcfg = Qwen25VLVisionConfig.from_hf(config["vision_config"])
    return WallOssEngine(cfg, text_config(config), vcfg, get_weight, names=set(names) if names is not None else None,
                         image_token_id=int(config.get("image_token_id", IMAGE_PAD_ID)), device=device, dtype=dtype,
                         max_prefix=max_seq_len - cfg.horizon, max_patches=max_patches)


# ----------------------------------------------------------------------------- host glue of one inference
def discretize_proprioception(norm_active: np.ndarray, state_bins: int = 256) -> str:
    """Normalised active proprioception values (in ``[-1, 1]``) -> space-joined bucket indices over ``state_bins``
    equal bins (the text form the policy was trained to read its state in)."""
    edges = np.linspace(-1, 1, state_bins + 1)[:-1]
    return " ".join(str(int(v)) for v in (np.digitize(norm_active, bins=edges) - 1).tolist())


def build_flow_prompt(instruction: str, camera_names: Sequence[str], dataset_name: str, delta_action: bool, propri_str: str, *,
                      style: str = "default") -> str:
    """The chat-formatted prompt up to (not including) the action placeholders: system prologue naming embodiment,
    cameras, control frequency and action space; one vision marker per camera; instruction; state string."""
    if style not in PROMPT_STYLES:
        raise ValueError(f"prompt style must be one of {PROMPT_STYLES}, got {style!r}")
    for c in camera_names:
        if c not in CAMERA_PROSE:
            raise ValueError(f"unknown camera {c!r}; known: {sorted(CAMERA_PROSE)}")
    marker = "<|vision_start|><|image_pad|><|vision_end|>"
    if style == "short":
        return f"<|im_start|>user\n{marker * len(camera_names)} {instruction}<|im_end|>\n<|im_start|>assistant\n"
    space = "Rel EEF" if delta_action else "Abs EEF"
    cams = ", ".join(CAMERA_PROSE[c] for c in camera_names)
    head = "<|im_start|>system\nYou are an embodied vision-language-action (VLA) model controlling the robot with language instructions.\n"
    if style == "multisuite":
        prologue = head + " Embodiment: Single Franka\n Camera Setup:" + "".join(f" {CAMERA_PROSE[c]}," for c in camera_names) \
            + f"\n Frequency: 10HZ\n Action Space: {space}\n<|im_end|>\n"
    elif style == "generic":
        prologue = ("<|im_start|>system\nYou are an embodied vision-language-action model controlling a robot with language "
                    f"instructions.\nCamera Setup: {cams}\nAction Space: {space}\n<|im_end|>\n")
    else:
        prologue = head + f" Embodiment: {dataset_name.split('_')[-1]}\n Camera Setup: {cams},\n Frequency: 32HZ\n Action Space: {space}\n<|im_end|>\n"
    user = "<|im_start|>user\nObservation:" + "".join(f" {CAMERA_PROSE[c]}: {marker}" for c in camera_names) + "\nInstruction:"
    tail = f"\nPredict the next action in robot action.\nProprioception: {propri_str}\n"
    return prologue + f"{user} {instruction}{tail}<|im_end|>\n" + "<|im_start|>assistant\n"


class Normalizer:
    """Per-dataset min / delta pairs of the ``normalizer_action.pth`` and ``normalizer_propri.pth`` sidecars:
    ``normalised = 2 * (raw - min) / delta - 1`` and back."""

    def __init__(self, action: Mapping, propri: Mapping, dataset_key: str, *, clamp: bool = True):
        for label, table in (("action", action), ("proprioception", propri)):
            for k in (f"min.{dataset_key}", f"delta.{dataset_key}"):
                if k not in table:
                    known = sorted({n.split(".", 1)[1] for n in table if "." in n})
                    raise RPUConfigError(f"{label} normalizer has no entry {k!r}; datasets: {known[:12]}")
        g = lambda t, k: torch.as_tensor(t[k], dtype=torch.float32)
        self.a_min, self.a_delta = g(action, f"min.{dataset_key}"), g(action, f"delta.{dataset_key}")
        self.p_min, self.p_delta = g(propri, f"min.{dataset_key}"), g(propri, f"delta.{dataset_key}")
        if bool((self.a_delta == 0).any()) or bool((self.p_delta == 0).any()):
            raise RPUConfigError("normalizer delta must be non-zero")
        self.dataset_key, self.clamp = dataset_key, clamp

    @classmethod
    def from_dir(cls, path: str, dataset_key: str, *, clamp: bool = True) -> "Normalizer":
        load = lambda n: torch.load(os.path.join(path, n), map_location="cpu", weights_only=True)
        a, p = load("normalizer_action.pth"), load("normalizer_propri.pth")
        unwrap = lambda t: t.get("state_dict", t) if isinstance(t, Mapping) else t
        return cls(unwrap(a), unwrap(p), dataset_key, clamp=clamp)

    def state_string(self, proprioception: torch.Tensor, state_mask: torch.Tensor, state_bins: int) -> str:
        raw = proprioception.float().reshape(-1)
        if raw.numel() != self.p_min.numel():
            raise ValueError(f"proprioception has {raw.numel()} entries, the normalizer {self.p_min.numel()}")
        norm = 2.0 * (raw - self.p_min) / self.p_delta - 1.0
        if self.clamp:
            norm = norm.clamp(-1.0, 1.0)
        return discretize_proprioception(norm[state_mask.reshape(-1).bool()].numpy(), state_bins)

    def denormalize(self, x: torch.Tensor) -> torch.Tensor:
        return (x.float() + 1.0) / 2.0 * self.a_delta + self.a_min

    def padding_action(self, horizon: int) -> torch.Tensor:
        """Normalised physical zero ``[horizon, action_dim]`` (the end point of inactive degrees of freedom)."""
        norm = 2.0 * (0.0 - self.a_min) / self.a_delta - 1.0
        if self.clamp:
            norm = norm.clamp(-1.0, 1.0)
        return (norm if norm.dim() == 2 else norm[None].expand(horizon, -1)).contiguous()


def expand_image_tokens(text: str, image_grid_thw: torch.Tensor, merge: int, token: str = "<|image_pad|>") -> str:
    """Repeat each image placeholder once per merged patch of its image, in order."""
    parts = text.split(token)
    if len(parts) - 1 != int(image_grid_thw.shape[0]):
        raise ValueError(f"{len(parts) - 1} image placeholders for {int(image_grid_thw.shape[0])} images")
    out = [parts[0]]
    for i, rest in enumerate(parts[1:]):
        out.append(token * int(int(image_grid_thw[i].prod()) // (merge * merge)))
        out.append(rest)
    return "".join(out)


__all__ = ["build_engine", "text_config", "action_config", "preflight", "build_flow_prompt", "discretize_proprioception",
           "Normalizer", "expand_image_tokens", "CAMERA_PROSE", "PROMPT_STYLES", "IMAGE_PAD_ID"]
