"""HunYuan embodied VLA (Hy-Embodied-0.5-VLA): host-side observation preprocessing.

Built here: everything between a raw observation (camera frames, instruction, proprioceptive state) and the tensors the
model consumes - image normalisation, prompt tokenisation, the prefix / suffix attention masks and position ids
(``preprocess``).  The HYViT2 tower is ``models/vision.py::HYViT2Encoder``; the twin-weight prefill and the action expert
are not built, so :class:`rhinoforge_b200.api.HyEmbodiedPolicy` still refuses to construct.
Reference counterpart: ``python/rpu_backend/adapters/hy_vla/preprocess.py``.
"""
from .preprocess import (CAMERA_ORDER, PrefixLayout, apply_visual_segment_mask, build_observation, make_att_2d_masks,
                         prefix_masks, prepare_images, prepare_language, prepare_state, resize_with_pad, sample_noise,
                         suffix_masks)

__all__ = ["CAMERA_ORDER", "PrefixLayout", "apply_visual_segment_mask", "build_observation", "make_att_2d_masks",
           "prefix_masks", "prepare_images", "prepare_language", "prepare_state", "resize_with_pad", "sample_noise",
           "suffix_masks"]
