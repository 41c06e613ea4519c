"""InternVLA-N1: the host-side goal glue between the language system and the navigation head.

Built: :mod:`goal_glue` (``vlm_tokens [B, 4, 3584] -> goal_embed [B, 1, 384]``, fp32 on the CPU as in the reference,
``python/rpu_backend/adapters/internvla_n1/goal_glue.py``).  The Qwen2.5-VL backbone it follows and the NextDiT /
NavDP heads it feeds are not built as policies."""
from .goal_glue import GoalGlue, TokenCompressor, build_goal_glue

__all__ = ["GoalGlue", "TokenCompressor", "build_goal_glue"]
