"""Policy facades of model families that this framework does not run yet.

The classes exist so that ``rpu_backend.api.HyEmbodiedPolicy`` imports and fails in a defined way: every
constructor path raises :class:`UnsupportedModelError` naming the family, what it would need and what is available
instead, before any checkpoint is read (the reference's facade: ``python/rpu_backend/api/hy_embodied.py``).
``WallOssPolicy``, ``Lingbot2Policy`` and ``RhinoVLAPolicy`` are not among them: they are built in
:mod:`rhinoforge_b200.api.wall_oss`, :mod:`rhinoforge_b200.api.lingbot2` and :mod:`rhinoforge_b200.api.rhinovla`.  The shared pieces those policies use - runtime-environment
validation, action de-normalisation, 6-D rotation decoding - are built (``_runtime_env``, ``action_denorm``,
``hy_action_decode``), and so are the towers they start from (Qwen2.5-VL ViT, SigLIP, the Qwen2.5 / Qwen3 decoder stack).
"""
from __future__ import annotations

from typing import Any

from .errors import UnsupportedModelError


def _facade(name: str, family: str, needs: str):
    def refuse(cls, *args: Any, **kwargs: Any):
        raise UnsupportedModelError(f"{family} is not built in this framework ({needs}); "
                                    "the policies that run today are Pi05Policy, Lingbot2Policy and WallOssPolicy")

    body = {
        "__doc__": f"{family}: defined, not runnable (see :mod:`rhinoforge_b200.api._unbuilt`).",
        "FAMILY": family,
        "from_checkpoint": classmethod(refuse),
        "from_pretrained": classmethod(refuse),
        "__init__": lambda self, *a, **k: refuse(type(self)),
    }
    return type(name, (), body)


HyEmbodiedPolicy = _facade("HyEmbodiedPolicy", "HunYuan embodied VLA (HYViT2 tower, twin-weight prefill, action expert)",
                           "needs the HYViT2 tower and row-routed twin weights")

__all__ = ["HyEmbodiedPolicy"]
