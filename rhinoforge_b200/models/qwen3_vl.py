"""Qwen3-VL: vision tower + M-RoPE text decoder with DeepStack injection.

Prefill does everything on the device: the text rows come from the embedding kernel, the merged
image embeddings are scattered over the image-placeholder rows, the three-axis positions feed the
interleaved M-RoPE of the QKV epilogue kernel, and the DeepStack features of vision layers
(5, 11, 17) are added to the visual rows after text layers 0, 1, 2 inside the native layer loop.
Decode continues with ``position = max position + 1`` on all three axes (the ``rope_delta`` rule).

Reference behaviour: ``python/rpu_backend/adapters/qwen3_vl/__init__.py:541,1211-1319`` (adapter,
masked scatter, rope index), ``adapters/qwen3_vl/text.py:52-55,87-160,371`` (DeepStack layer map,
M-RoPE tables), ``src/fused/rpu_qwen3_model.h:3594-3623`` (DeepStack add after the MLP),
``src/ops/rpu_mrope.cpp:37-124`` (interleaved axis select).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch

from ..ops import kernels as K
from ..runtime.engine import DecoderEngine
from ..runtime.errors import RPUBackendError, UnsupportedModelError
from .decoder import DecoderConfig
from .vision import Qwen3VLVisionConfig, Qwen3VLVisionEncoder

TEXT_PROFILES = {(2048, 6144, 28, 8): "qwen3-vl-2b", (2560, 9728, 36, 8): "qwen3-vl-4b",
                 (4096, 12288, 36, 8): "qwen3-vl-8b", (5120, 25600, 64, 8): "qwen3-vl-32b"}
VISION_PROFILE = dict(hidden_size=1024, intermediate_size=4096, depth=24, num_heads=16, patch_size=16,
                      temporal_patch_size=2, spatial_merge_size=2)


def _cfg_get(c, k, d=None):
    return c.get(k, d) if isinstance(c, dict) else getattr(c, k, d)


def text_config_of(hf_config) -> DecoderConfig:
    tc = _cfg_get(hf_config, "text_config", hf_config)
    cfg = DecoderConfig.from_hf(tc)
    if cfg.mrope_section is None:
        raise UnsupportedModelError("Qwen3-VL text config carries no mrope_section")
    return cfg


def preflight(hf_config, *, strict: bool = True) -> None:
    """Config-only admission (nothing is loaded or moved before this passes)."""
    cfg = text_config_of(hf_config)
    vc = _cfg_get(hf_config, "vision_config")
    if strict:
        if cfg.profile() not in TEXT_PROFILES:
            raise UnsupportedModelError(f"Qwen3-VL text profile {cfg.profile()} is not admitted; known: {sorted(TEXT_PROFILES)}")
        for k, v in VISION_PROFILE.items():
            if _cfg_get(vc, k) != v:
                raise UnsupportedModelError(f"Qwen3-VL vision_config.{k}={_cfg_get(vc, k)!r}, expected {v!r}")
    if _cfg_get(vc, "hidden_act", "gelu_pytorch_tanh") not in ("gelu_pytorch_tanh", "gelu"):
        raise UnsupportedModelError("Qwen3-VL vision activation must be gelu_pytorch_tanh or gelu")


def rope_index(token_types: Sequence[int], image_grids: Sequence[Sequence[int]], merge: int,
               video_grids: Sequence[Sequence[int]] = ()) -> torch.Tensor:
    """Three-axis (t, h, w) positions ``[3, L]`` for one sequence.

    ``token_types[i]`` is 0 for text, 1 for an image placeholder row and 2 for a video-frame
    placeholder row; every maximal run of one non-zero type consumes the next grid ``(t, h, w)`` (in
    patches) of that kind -- a video of ``t`` frames counts as ``t`` grids ``(1, h, w)``, one per
    timestamp-separated run -- and, when images follow each other without a separator token, as many
    further grids as it takes to cover the run.  Text advances all three axes together; a vision run occupies
    ``t = start``, ``h = start + row``, ``w = start + col`` and the following text resumes at
    ``start + max(h, w) / merge``."""
    frames = [(1, int(h), int(w)) for t, h, w in video_grids for _ in range(int(t))]
    queues = {1: list(image_grids), 2: frames}
    out: List[torch.Tensor] = []
    cur, i, L = 0, 0, len(token_types)
    while i < L:
        j = i
        kind = token_types[i]
        while j < L and token_types[j] == kind:
            j += 1
        if kind == 0:
            out.append(torch.arange(cur, cur + (j - i)).view(1, -1).expand(3, -1))
            cur += j - i
        else:
            left = j - i
            while left > 0:
                if not queues[kind]:
                    raise RPUBackendError("more vision placeholder rows than the grids cover")
                t, h, w = (int(v) for v in queues[kind].pop(0))
                gh, gw = h // merge, w // merge
                if t * gh * gw > left:
                    raise RPUBackendError(f"vision placeholder run of {j - i} rows does not match grid {(t, h, w)}")
                pw = torch.arange(cur, cur + gw).repeat(gh * t)
                ph = torch.arange(cur, cur + gh).repeat_interleave(gw * t)
                pt = torch.full((t * gh * gw,), cur)
                out.append(torch.stack((pt, ph, pw)))
                cur += max(h, w) // merge
                left -= t * gh * gw
        i = j
    return torch.cat(out, 1).to(torch.int32)


class Qwen3VLEngine:
    """Vision encoder + decoder engine.  ``get_weight(name)`` serves Hugging Face checkpoint names
    (``model.visual.*``, ``model.language_model.*``, ``lm_head.weight``)."""

    def __init__(self, hf_config, get_weight: Callable[[str], torch.Tensor], *, device="cuda", dtype=torch.float16,
                 max_seq_len: int = 4096, max_batch: int = 1, max_patches: int = 4096, max_prefill_tokens: int = 4096,
                 tp=None, quant: Optional[str] = None, strict_profiles: bool = False, names: Optional[set] = None):
        preflight(hf_config, strict=strict_profiles)
        self.hf_config = hf_config
        self.cfg = text_config_of(hf_config)
        vc = _cfg_get(hf_config, "vision_config")
        self.vcfg = Qwen3VLVisionConfig.from_hf(vc)
        self.image_token_id = _cfg_get(hf_config, "image_token_id", 151655)
        self.video_token_id = _cfg_get(hf_config, "video_token_id", 151656)
        self.device, self.dtype = torch.device(device), dtype

        def text_get(name: str) -> torch.Tensor:
            if name.startswith("model."):
                return get_weight("model.language_model." + name[len("model."):])
            return get_weight(name)
        if names is not None:
            text_get.names = {("model." + n[len("model.language_model."):]) if n.startswith("model.language_model.") else n
                              for n in names}
        scale = getattr(get_weight, "scale", None)
        if scale is not None:
            text_get.scale = lambda n: scale("model.language_model." + n[len("model."):] if n.startswith("model.") else n)
        kw = dict(tp=tp) if tp is not None else {}
        self.text = DecoderEngine(self.cfg, text_get, device=device, dtype=dtype, max_batch=max_batch,
                                  max_seq_len=max_seq_len, max_prefill_tokens=max_prefill_tokens, quant=quant, **kw)

        class _VisionSD(dict):
            def __missing__(_, key):          # lazy view over the getter: the encoder asks by full name
                return get_weight(key)
        self.vision = Qwen3VLVisionEncoder(self.vcfg, _VisionSD(), prefix="model.visual.", device=device, dtype=dtype,
                                           max_patches=max_patches)
        if len(self.vcfg.deepstack_visual_indexes) > self.cfg.num_layers:
            raise UnsupportedModelError("more DeepStack taps than text layers")

    # ------------------------------------------------------------------ multimodal prefill
    @torch.no_grad()
    def prepare(self, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor] = None, image_grid_thw=None):
        """Build ``(inputs_embeds [L,H], positions3 [3,L], deepstack)`` for one sequence."""
        ids = input_ids.flatten().to("cpu")
        is_vis = ids == self.image_token_id
        if bool((ids == self.video_token_id).any()):
            raise RPUBackendError("video placeholders are not supported by this entry point")
        grids = [] if image_grid_thw is None else [tuple(int(v) for v in g) for g in torch.as_tensor(image_grid_thw).tolist()]
        pos3 = rope_index(is_vis.to(torch.int32).tolist(), grids, self.vcfg.spatial_merge_size)
        ids_d = ids.to(self.device, torch.int32)
        embeds = torch.empty((ids.numel(), self.cfg.hidden_size), dtype=self.dtype, device=self.device)
        K.embedding(self.text.embed, ids_d, out=embeds, scale=self.cfg.embed_scale, row_scale=self.text.embed_scale_rows)
        deep = None
        if pixel_values is not None:
            img, feats = self.vision(pixel_values, grids)
            rows = is_vis.nonzero().flatten()
            if rows.numel() != img.shape[0]:
                raise RPUBackendError(f"{rows.numel()} image placeholder tokens but {img.shape[0]} image embeddings")
            K.scatter_rows(embeds, img, rows.to(self.device, torch.int32))
            deep = (rows, feats) if feats else None     # a tower without DeepStack taps (Qwen3.5) adds nothing to the text layers
        elif bool(is_vis.any()):
            raise RPUBackendError("input_ids contain image placeholders but no pixel_values were given")
        return embeds, pos3, deep

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor] = None, image_grid_thw=None, *,
                return_logits: bool = False):
        """Start sequence 0 from empty with a (possibly multimodal) prompt; returns the greedy next token."""
        self.text.reset()
        return self.extend(input_ids, pixel_values, image_grid_thw, return_logits=return_logits)

    @torch.no_grad()
    def extend(self, input_ids: torch.Tensor, pixel_values=None, image_grid_thw=None, *, return_logits: bool = False):
        ids = input_ids.flatten()
        start = self.text.cache.lengths[0]
        if start == 0 or pixel_values is not None:
            embeds, pos3, deep = self.prepare(ids, pixel_values, image_grid_thw)
            if start:
                pos3 = pos3 + int(self._next_pos)
            self._next_pos = int(pos3.max()) + 1
            return self.text.extend([ids], return_logits=return_logits, inputs_embeds=[embeds], positions3=[pos3],
                                    deepstack=[deep] if deep is not None else None)
        # text continuation after an image: positions run on from the stored next position
        pos3 = (torch.arange(ids.numel(), dtype=torch.int32) + int(self._next_pos)).view(1, -1).expand(3, -1)
        self._next_pos = int(pos3.max()) + 1
        return self.text.extend([ids], return_logits=return_logits, positions3=[pos3])

    @torch.no_grad()
    def prefill_batch(self, input_ids: Sequence[torch.Tensor], pixel_values: Sequence[torch.Tensor],
                      image_grid_thw: Sequence, *, return_logits: bool = False):
        """Start sequences ``0..B-1`` from empty, each with its own multimodal prompt: the images of the whole batch go
        through the vision tower as ONE packed pass, every sequence gets its own embeddings, three-axis positions
        and DeepStack rows, and the text decoder prefills all of them as one packed varlen launch.  Returns the greedy
        next token of every sequence (with ``return_logits`` also the last-row logits)."""
        self.text.reset()
        B = len(input_ids)
        merge2 = self.vcfg.spatial_merge_size ** 2
        grids = [[tuple(int(v) for v in g) for g in torch.as_tensor(gr).tolist()] for gr in image_grid_thw]
        img, feats = self.vision(torch.cat([p.to(self.device) for p in pixel_values]), [g for gr in grids for g in gr])
        embeds, pos3s, deeps, o = [], [], [], 0
        for s in range(B):
            ids = input_ids[s].flatten().to("cpu")
            is_vis = ids == self.image_token_id
            n_img = sum(t * h * w for t, h, w in grids[s]) // merge2
            rows = is_vis.nonzero().flatten()
            if rows.numel() != n_img:
                raise RPUBackendError(f"sequence {s}: {rows.numel()} image placeholder tokens but {n_img} image embeddings")
            e = torch.empty((ids.numel(), self.cfg.hidden_size), dtype=self.dtype, device=self.device)
            K.embedding(self.text.embed, ids.to(self.device, torch.int32), out=e, scale=self.cfg.embed_scale,
                        row_scale=self.text.embed_scale_rows)
            K.scatter_rows(e, img[o:o + n_img], rows.to(self.device, torch.int32))
            embeds.append(e)
            pos3s.append(rope_index(is_vis.to(torch.int32).tolist(), grids[s], self.vcfg.spatial_merge_size))
            deeps.append((rows, [f[o:o + n_img] for f in feats]) if feats else None)
            o += n_img
        self._next_pos = max(int(p.max()) for p in pos3s) + 1
        return self.text.extend([t.flatten() for t in input_ids], return_logits=return_logits, inputs_embeds=embeds,
                                positions3=pos3s, deepstack=deeps if any(d is not None for d in deeps) else None)

    def decode(self, n_steps: int, **kw) -> torch.Tensor:
        out = self.text.decode(n_steps, **kw)
        self._next_pos += n_steps
        return out

    @torch.no_grad()
    def generate(self, input_ids, pixel_values=None, image_grid_thw=None, max_new_tokens: int = 16) -> torch.Tensor:
        first = self.prefill(input_ids, pixel_values, image_grid_thw)
        if max_new_tokens <= 1:
            return first[:, None]
        rest = self.decode(max_new_tokens - 1)
        self.text.check_status()
        return torch.cat((first[:, None], rest), 1)

    def close(self) -> None:
        self.vision.close()
        self.text.close()
