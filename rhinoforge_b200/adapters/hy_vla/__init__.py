"""HunYuan embodied VLA (Hy-Embodied-0.5-VLA): observation preprocessing and the runtime build.

Built here: everything between a raw observation (camera frames, instruction, proprioceptive state) and the tensors the
model consumes - image normalisation, prompt tokenisation, the prefix / suffix attention masks and position ids
(``preprocess``) - and ``runtime``: checkpoint -> engine (HYViT2 tower + merger, twin-weight VLM prefill, action expert:
:mod:`rhinoforge_b200.models.hyvla`) and the action-chunk pipeline behind :class:`rhinoforge_b200.api.HyEmbodiedPolicy`.
Reference counterparts: ``python/rpu_backend/adapters/hy_vla/preprocess.py``, ``runtime.py``, ``weights.py``.
"""
from .preprocess import (CAMERA_ORDER, PrefixLayout, apply_visual_segment_mask, build_observation, make_att_2d_masks,
                         prefix_masks, prepare_images, prepare_language, prepare_state, resize_with_pad, sample_noise,
                         suffix_masks)

__all__ = ["CAMERA_ORDER", "PrefixLayout", "apply_visual_segment_mask", "build_observation", "make_att_2d_masks",
           "prefix_masks", "prepare_images", "prepare_language", "prepare_state", "resize_with_pad", "sample_noise",
           "suffix_masks"]
