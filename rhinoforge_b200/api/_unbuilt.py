"""Policy facades of model families that this framework does not run yet.

None is left: ``Pi05Policy``, ``Lingbot2Policy``, ``WallOssPolicy``, ``HyEmbodiedPolicy`` and ``RhinoVLAPolicy`` are built
in :mod:`rhinoforge_b200.api.policy`, ``lingbot2``, ``wall_oss``, ``hy_embodied`` and ``rhinovla``.  The factory stays for a
family whose facade should import and fail in a defined way - every constructor path raising
:class:`UnsupportedModelError` that names the family and what it would need - before its runtime exists.
"""
from __future__ import annotations

from typing import Any

from .errors import UnsupportedModelError


def unbuilt_facade(name: str, family: str, needs: str):
    def refuse(cls, *args: Any, **kwargs: Any):
        raise UnsupportedModelError(f"{family} is not built in this framework ({needs})")

    body = {
        "__doc__": f"{family}: defined, not runnable (see :mod:`rhinoforge_b200.api._unbuilt`).",
        "FAMILY": family,
        "from_checkpoint": classmethod(refuse),
        "from_pretrained": classmethod(refuse),
        "__init__": lambda self, *a, **k: refuse(type(self)),
    }
    return type(name, (), body)


__all__ = ["unbuilt_facade"]
