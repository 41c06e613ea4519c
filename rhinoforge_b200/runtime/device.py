"""Device-string handling: ``"rpu"`` (and ``"rpu:0"``) name the current CUDA device.

The reference accepts only device index 0 (``python/rpu_backend/runtime/device.py:37-41``); here an
index selects the CUDA ordinal, and tensor-parallel ranks use their local GPU."""
from __future__ import annotations

from typing import Union


def resolve_device(device: Union[str, "object", None]):
    import torch
    if device is None:
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    if isinstance(device, str):
        name = device.strip().lower()
        if name == "rpu" or name.startswith("rpu:"):
            idx = int(name.split(":", 1)[1]) if ":" in name else None
            if not torch.cuda.is_available():
                raise RuntimeError("device 'rpu' needs a CUDA device (B200); none is available")
            return torch.device("cuda", torch.cuda.current_device() if idx is None else idx)
        return torch.device(device)
    if getattr(device, "type", None) in ("rpu", "privateuseone"):
        idx = getattr(device, "index", None)
        return torch.device("cuda", torch.cuda.current_device() if idx is None else idx)
    return torch.device(device)


def is_rpu_request(device) -> bool:
    if device is None:
        return False
    name = device if isinstance(device, str) else getattr(device, "type", "")
    return str(name).lower().startswith(("rpu", "privateuseone"))
