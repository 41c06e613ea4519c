"""Gemma4 text decoder: the host-side planning modules.

Gemma4 mixes two layer geometries - sliding-window layers (head_dim 256) and global layers (head_dim 512, proportional
RoPE) - and lets its last layers reuse the K/V of an earlier layer of the same type.  Built here: the per-layer geometry
table with its graph-signature encoding (``geometry``), the paged KV plan with the mandatory source map
(``cache_plan``) and the sliding-window mask oracle (``windowed_mask``).  The decoder runs on
:class:`rhinoforge_b200.models.gemma4.Gemma4Engine` (``runtime.Gemma4Adapter`` / ``Gemma4Handle``, resolved lazily).
Reference counterparts: ``python/rpu_backend/adapters/gemma4/{geometry,cache_plan,_mask}.py``.
"""
from .cache_plan import cache_plan, layer_slot_shape, windowed_mask
from .geometry import (GLOBAL_LAYER_TYPE, SLIDING_LAYER_TYPE, LayerGeom, geometry_dyn_dims, geometry_hash,
                       layer_geometry, max_head_dim, max_num_kv_heads, native_layer_arrays)



def __getattr__(name):
    if name in ("Gemma4Adapter", "Gemma4Handle"):
        from . import runtime
        return getattr(runtime, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = ["Gemma4Adapter", "Gemma4Handle", "LayerGeom", "layer_geometry", "native_layer_arrays", "geometry_hash", "geometry_dyn_dims", "max_head_dim",
           "max_num_kv_heads", "cache_plan", "layer_slot_shape", "windowed_mask", "GLOBAL_LAYER_TYPE",
           "SLIDING_LAYER_TYPE"]
