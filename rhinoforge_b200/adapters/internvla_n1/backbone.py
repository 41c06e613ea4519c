"""InternVLA-N1 System-2: the Qwen2.5-VL backbone read at its latent-query positions.

System-2 hands System-1 ``vlm_tokens = hidden_states[-1][:, -4:, :]``: the final-layer hidden state (after the final
RMSNorm) of the last four positions, where the prompt carries the latent queries.  :class:`Qwen25VLBackbone` runs the
multimodal prefill on :class:`rhinoforge_b200.models.qwen25_vl.Qwen25VLEngine` (windowed ViT, chunked M-RoPE, QKV bias) and
normalises only those rows.  ``forward_embeds`` serves callers that assemble the input embeddings themselves (image rows
scattered, latent queries appended) and pass their three-axis positions.

Reference: ``python/rpu_backend/adapters/internvla_n1/backbone.py:1-24`` (what is read and where),
``python/rpu_backend/adapters/internvla_n1/vision.py`` (tower builder).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Mapping, Optional

import torch

from ...api.errors import UnsupportedModelError
from ...models.qwen25_vl import Qwen25VLEngine, qwen25_text_config
from ...models.qwen25_vl_vision import Qwen25VLVisionConfig
from .._assets import verify_asset_manifest

NUM_LATENT = 4
PROFILE = dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, num_hidden_layers=28)


def _get(c, k, d=None):
    return c.get(k, d) if isinstance(c, Mapping) else getattr(c, k, d)


def preflight(hf_config, *, strict: bool = True) -> None:
    tc = _get(hf_config, "text_config", None) or hf_config
    if strict:
        bad = {k: _get(tc, k) for k, v in PROFILE.items() if _get(tc, k) != v}
        if bad:
            raise UnsupportedModelError(f"InternVLA-N1 System-2 expects the Qwen2.5-VL-7B geometry {PROFILE}; this config has {bad}")
    if _get(hf_config, "vision_config", None) is None:
        raise UnsupportedModelError("the System-2 checkpoint has no vision_config")


class Qwen25VLBackbone:
    def __init__(self, engine: Qwen25VLEngine, *, num_latent: int = NUM_LATENT):
        self.engine, self.num_latent = engine, num_latent

    def _tail(self, n_rows: int) -> torch.Tensor:
        from ...ops import kernels as K
        t = self.engine.text
        if n_rows < self.num_latent:
            raise ValueError(f"the prompt has {n_rows} rows, fewer than the {self.num_latent} latent queries")
        if n_rows > t.max_tokens:
            raise ValueError(f"{n_rows} rows exceed one prefill launch ({t.max_tokens}): build with a larger max_prefill_tokens")
        rows = t.hidden[n_rows - self.num_latent:n_rows]
        out = K.rmsnorm(rows, t.final_norm, self.engine.cfg.rms_eps)
        t.check_status()
        return out.float()[None]

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor] = None, image_grid_thw=None) -> torch.Tensor:
        """``vlm_tokens [1, 4, hidden]`` fp32 on the device."""
        ids = input_ids.reshape(-1)
        self.engine.prefill(ids, pixel_values, image_grid_thw)
        return self._tail(int(ids.numel()))

    @torch.no_grad()
    def forward_embeds(self, inputs_embeds: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        """``inputs_embeds [1, L, hidden]`` (or ``[L, hidden]``), ``position_ids [3, 1, L]`` (or ``[3, L]``) -> ``[1, 4, hidden]``."""
        emb = inputs_embeds.reshape(-1, inputs_embeds.shape[-1])
        pos3 = position_ids.reshape(3, -1).to(torch.int32)
        t = self.engine.text
        t.reset()
        ids = torch.zeros(emb.shape[0], dtype=torch.int32)
        t.extend([ids], inputs_embeds=[emb.to(self.engine.device, self.engine.dtype)], positions3=[pos3])
        return self._tail(int(emb.shape[0]))

    __call__ = forward

    def close(self) -> None:
        self.engine.close()


def build_qwen25vl_backbone(model_dir: str, *, get_weight: Optional[Callable[[str], torch.Tensor]] = None, hf_config=None,
                            asset_manifest: Optional[Mapping] = None, strict: bool = True, max_seq_len: int = 4096,
                            max_patches: int = 4096, device="cuda", dtype=torch.float16) -> Qwen25VLBackbone:
    """``model_dir``: a Hugging Face Qwen2.5-VL checkpoint directory (``config.json`` + safetensors); ``get_weight`` /
    ``hf_config`` replace the files for in-memory weights."""
    if hf_config is None:
        with open(os.path.join(model_dir, "config.json")) as f:
            hf_config = json.load(f)
    preflight(hf_config, strict=strict)
    if get_weight is None:
        from ...api._loading import checkpoint_tensor_getter
        import glob
        verify_asset_manifest(sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))), asset_manifest)
        get_weight = checkpoint_tensor_getter(model_dir)
    names = getattr(get_weight, "names", None)
    nested = names is None or any(n.startswith("model.language_model.") for n in names)

    def text_get(name: str) -> torch.Tensor:
        if nested and name.startswith("model."):
            return get_weight("model.language_model." + name[len("model."):])
        return get_weight(name)
    vprefix = "model.visual." if nested else "visual."

    class _Vision(dict):
        def __missing__(self, key):
            return get_weight(vprefix + key)

        def __contains__(self, key):
            return names is None or (vprefix + key) in names

        def get(self, key, default=None):
            try:
                return self[key]
            except KeyError:
                return default
    tc = _get(hf_config, "text_config", None) or hf_config
    if isinstance(tc, Mapping):                                  # a plain config.json: the decoder reader takes attributes
        from types import SimpleNamespace
        tc = SimpleNamespace(**tc)
        if getattr(tc, "rope_parameters", None) is None and getattr(tc, "rope_scaling", None) is not None:
            tc.rope_parameters = {**tc.rope_scaling, "rope_theta": getattr(tc, "rope_theta", 1e6)}
    cfg = qwen25_text_config(tc)
    vcfg = Qwen25VLVisionConfig.from_hf(_get(hf_config, "vision_config"))
    eng = Qwen25VLEngine(cfg, vcfg, text_get, _Vision(), image_token_id=int(_get(hf_config, "image_token_id", 151655)), device=device,
                         dtype=dtype, max_seq_len=max_seq_len, max_patches=max_patches, max_prefill_tokens=max_seq_len)
    return Qwen25VLBackbone(eng)


__all__ = ["Qwen25VLBackbone", "build_qwen25vl_backbone", "preflight", "NUM_LATENT"]
