"""InternVLA-N1: the pieces between the language system and the navigation actions.

* :mod:`goal_glue` - ``vlm_tokens [B, 4, 3584] -> goal_embed [B, 1, 384]``, fp32 on the CPU as in the reference
  (``python/rpu_backend/adapters/internvla_n1/goal_glue.py``);
* :mod:`nextdit` - the Lumina NextDiT trajectory head on the accelerator (``build_nextdit_runtime``);
* :mod:`backbone` - System-2: the Qwen2.5-VL backbone read at its four latent-query positions (``build_qwen25vl_backbone``);
* :mod:`rgbd` - the RGB-D encoder of System-1 (two DINOv2 ViT-S towers + a perceiver; ``build_rgbd_encoder``);
* the NavDP diffusion head lives in :mod:`rhinoforge_b200.adapters.navdp` (its checkpoint is a bundle of its own).

The NextDiT names resolve lazily so that importing the goal glue does not load the device runtime."""
from .goal_glue import GoalGlue, TokenCompressor, build_goal_glue

_LAZY = {"NextDiTRuntime": ".nextdit", "build_nextdit_runtime": ".nextdit", "Qwen25VLBackbone": ".backbone",
         "build_qwen25vl_backbone": ".backbone", "build_rgbd_encoder": ".rgbd"}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        return getattr(importlib.import_module(_LAZY[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = ["GoalGlue", "TokenCompressor", "build_goal_glue", "NextDiTRuntime", "build_nextdit_runtime", "Qwen25VLBackbone",
           "build_qwen25vl_backbone", "build_rgbd_encoder"]
