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


def _field(cfg: Any, name: str, default: Any = None) -> Any:
    return cfg.get(name, default) if isinstance(cfg, dict) else getattr(cfg, name, default)


def layer_geometry(text_config: Any) -> List[LayerGeom]:
    """The table for a ``Gemma4TextConfig`` or the plain ``text_config`` dict of a ``config.json``."""
    n_layers = int(_field(text_config, "num_hidden_layers"))
    types = list(_field(text_config, "layer_types"))
    if len(types) != n_layers:
        raise ValueError(f"layer_types length {len(types)} != num_hidden_layers {n_layers}")
    first_shared = n_layers - int(_field(text_config, "num_kv_shared_layers", 0) or 0)
    hd_sliding = int(_field(text_config, "head_dim"))
    hd_global = int(_field(text_config, "global_head_dim") or hd_sliding)
    n_q = int(_field(text_config, "num_attention_heads"))
    n_kv = int(_field(text_config, "num_key_value_heads"))
    n_kv_global = _field(text_config, "num_global_key_value_heads")
    k_is_v = bool(_field(text_config, "attention_k_eq_v", False))
    window = _field(text_config, "sliding_window")

    source_of_type: Dict[str, int] = {t: i for i, t in enumerate(types[:first_shared])}    # last owner wins
    table: List[LayerGeom] = []
    for i, t in enumerate(types):
        glob = t == GLOBAL_LAYER_TYPE
        shared = i >= first_shared
        if shared and t not in source_of_type:
            raise ValueError(f"layer {i} ({t}) is KV-shared but no non-shared source layer of that type exists in "
                             f"[0,{first_shared})")
        table.append(LayerGeom(
            idx=i, layer_type=t, is_global=glob, head_dim=hd_global if glob else hd_sliding, num_q_heads=n_q,
            num_kv_heads=int(n_kv_global) if (glob and k_is_v and n_kv_global) else n_kv,
            rope_type="proportional" if glob else "default",
            sliding_window=None if glob or not window else int(window),
            is_kv_shared=shared, kv_source_layer=source_of_type[t] if shared else i, has_kv_proj=not shared))
    return table


def native_layer_arrays(geo: List[LayerGeom]) -> Dict[str, List[int]]:
    """The per-layer integer arrays a native stack takes verbatim."""
    return {"layer_type_ids": [g.layer_type_id for g in geo], "head_dim_per_layer": [g.head_dim for g in geo],
            "num_kv_heads_per_layer": [g.num_kv_heads for g in geo], "kv_source_layer": [g.kv_source_layer for g in geo],
            "is_kv_shared": [int(g.is_kv_shared) for g in geo], "has_kv_proj": [int(g.has_kv_proj) for g in geo]}


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
