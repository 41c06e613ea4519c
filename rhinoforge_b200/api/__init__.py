"""Public API facades (lazy: importing this package does not import a model family)."""
from .errors import (RPUBackendError, RPUConfigError, RPUSingleHandleError, RPUUnsupportedDtypeError,  # noqa: F401
                     SPMExhaustionError, UnsupportedModelError, WeightShapeMismatchError)

_LAZY = {
    "RPUModelForCausalLM": ("causal_lm", "RPUModelForCausalLM"),
    "RPUCache": ("cache", "RPUCache"),
    "RPUModelForConditionalGeneration": ("conditional_generation", "RPUModelForConditionalGeneration"),
    "Qwen3_5Cache": ("qwen3_5_cache", "Qwen3_5Cache"),
    "Pi05Policy": ("policy", "Pi05Policy"),
    "WallOssPolicy": ("wall_oss", "WallOssPolicy"),
    "WallOssActionOutput": ("wall_oss", "WallOssActionOutput"),
    "Lingbot2Policy": ("lingbot2", "Lingbot2Policy"),
    "Lingbot2ActionOutput": ("lingbot2", "Lingbot2ActionOutput"),
    "HyEmbodiedPolicy": ("hy_embodied", "HyEmbodiedPolicy"),
    "HyEmbodiedActionOutput": ("hy_embodied", "HyEmbodiedActionOutput"),
    "RhinoVLAPolicy": ("rhinovla", "RhinoVLAPolicy"),
}


def __getattr__(name: str):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = ["RPUBackendError", "RPUConfigError", "UnsupportedModelError", "RPUUnsupportedDtypeError",
           "RPUSingleHandleError", "SPMExhaustionError", "WeightShapeMismatchError", *_LAZY]
