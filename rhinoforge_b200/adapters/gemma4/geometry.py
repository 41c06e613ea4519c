"""Per-layer geometry of a Gemma4 text decoder and its encoding into a graph signature.

Standard library only, so that it can be imported and checked without PyTorch or the native library.  Two consumers read
the same table: the per-layer integer arrays a native stack is configured with, and the graph-signature key - a captured
graph depends on every layer's width and K/V routing, none of which the base signature (rows x hidden, layer count)
carries, so the geometry is folded into two extra dynamic dimensions.  Reference behaviour:
``python/rpu_backend/adapters/gemma4/geometry.py:27-165``.

K/V sharing: the last ``num_kv_shared_layers`` layers have no k / v / k-norm weights; each reads the cache slot of the
last *non-shared* layer of its own type.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional

GLOBAL_LAYER_TYPE = "full_attention"
SLIDING_LAYER_TYPE = "sliding_attention"


@dataclass(frozen=True)
class LayerGeom:
    idx: int
    layer_type: str
    is_global: bool
    head_dim: int                     # sliding layers: head_dim; global layers: global_head_dim
    num_q_heads: int
    num_kv_heads: int
    rope_type: str                    # "default" on sliding layers, "proportional" on global ones
    sliding_window: Optional[int]     # None on global layers
    is_kv_shared: bool
    kv_source_layer: int              # the layer whose cache slot attention reads; idx itself when not shared
    has_kv_proj: bool

    @property
    def layer_type_id(self) -> int:
        """0 sliding, 1 global."""
        return int(self.is_global)

    def signature_fields(self) -> Iterable[int]:
        """What changes the launched kernels or their wiring, in hashing order."""
        return (self.head_dim, self.num_kv_heads, self.layer_type_id, int(self.is_kv_shared), self.kv_source_layer)


class _Cfg:
    """Uniform reader over a config object or the plain dict of a ``config.json``."""

    def __init__(self, raw: Any):
        self._get = raw.get if isinstance(raw, dict) else (lambda k, d=None: getattr(raw, k, d))

    def __call__(self, key: str, default: Any = None) -> Any:
        return self._get(key, default)

    def integer(self, key: str, default: int = 0) -> int:
        return int(self._get(key, None) or default)


def layer_geometry(text_config: Any) -> List[LayerGeom]:
    """The table for a ``Gemma4TextConfig`` or the plain ``text_config`` dict of a ``config.json``."""
    cfg = _Cfg(text_config)
    depth = cfg.integer("num_hidden_layers")
    kinds = list(cfg("layer_types"))
    if len(kinds) != depth:
        raise ValueError(f"layer_types length {len(kinds)} != num_hidden_layers {depth}")
    owners_end = depth - cfg.integer("num_kv_shared_layers")
    width = {False: cfg.integer("head_dim")}
    width[True] = cfg.integer("global_head_dim", width[False])
    kv_heads = {False: cfg.integer("num_key_value_heads")}
    kv_heads[True] = (cfg.integer("num_global_key_value_heads", kv_heads[False])
                      if cfg("attention_k_eq_v", False) else kv_heads[False])
    window = cfg.integer("sliding_window") or None
    q_heads = cfg.integer("num_attention_heads")

    donor: Dict[str, int] = {}                      # per layer type: the last layer that still owns its K/V
    for i in range(owners_end):
        donor[kinds[i]] = i
    table: List[LayerGeom] = []
    for i, kind in enumerate(kinds):
        wide, borrows = kind == GLOBAL_LAYER_TYPE, i >= owners_end
        if borrows and kind not in donor:
            raise ValueError(f"layer {i} ({kind}) is KV-shared but no non-shared source layer of that type exists in "
                             f"[0,{owners_end})")
        table.append(LayerGeom(i, kind, wide, width[wide], q_heads, kv_heads[wide],
                               "proportional" if wide else "default", None if wide else window,
                               borrows, donor[kind] if borrows else i, not borrows))
    return table


_NATIVE_COLUMNS = (("layer_type_ids", "layer_type_id"), ("head_dim_per_layer", "head_dim"),
                   ("num_kv_heads_per_layer", "num_kv_heads"), ("kv_source_layer", "kv_source_layer"),
                   ("is_kv_shared", "is_kv_shared"), ("has_kv_proj", "has_kv_proj"))


def native_layer_arrays(geo: List[LayerGeom]) -> Dict[str, List[int]]:
    """The per-layer integer arrays a native stack takes verbatim."""
    return {column: [int(getattr(g, attr)) for g in geo] for column, attr in _NATIVE_COLUMNS}


cpp_layer_arrays = native_layer_arrays          # the reference's name for the same table


def max_head_dim(geo: List[LayerGeom]) -> int:
    """Scratch buffers are sized for the widest layer."""
    return max(g.head_dim for g in geo)


def max_num_kv_heads(geo: List[LayerGeom]) -> int:
    return max(g.num_kv_heads for g in geo)


_FNV_OFFSET, _FNV_PRIME = 0xCBF29CE484222325, 0x100000001B3


def geometry_hash(geo: List[LayerGeom]) -> int:
    """Order-sensitive 64-bit FNV-1a over every layer's signature fields, cut to 63 bits so that it is a valid
    non-negative signed dimension."""
    h = _FNV_OFFSET
    for g in geo:
        for v in g.signature_fields():
            h = ((h ^ (int(v) & 0xFFFFFFFF)) * _FNV_PRIME) & 0xFFFFFFFFFFFFFFFF
    return h & 0x7FFFFFFFFFFFFFFF


def geometry_dyn_dims(geo: List[LayerGeom]) -> List[int]:
    """``[num_layers, geometry_hash]`` - appended to a graph signature's dynamic dimensions, so that a different
    geometry can never replay this one's graph."""
    return [len(geo), geometry_hash(geo)]


__all__ = ["LayerGeom", "layer_geometry", "native_layer_arrays", "cpp_layer_arrays", "max_head_dim", "max_num_kv_heads",
           "geometry_hash", "geometry_dyn_dims", "GLOBAL_LAYER_TYPE", "SLIDING_LAYER_TYPE"]
