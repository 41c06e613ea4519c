"""Mixed-width paged KV plan for Gemma4, with the source map that K/V sharing makes mandatory.

A shared layer *reads another layer's slot*, which a per-layer maximum-width cache cannot express; the plan therefore
always yields ``source_map[i]`` (the layer whose slot layer ``i``'s attention reads) and allocates only for owners.
Slots use this framework's paged layout - per owner ``[2, pages, kv_heads, 16, head_dim]``, 16 tokens per page - and,
unlike a dense cache, a sliding layer needs pages only for its window (plus one page of slack for the page being
written), which on a 128 k context is most of the saving.  Reference behaviour (dense 7-D slots):
``python/rpu_backend/adapters/gemma4/cache_plan.py:33-121``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

PAGE_TOKENS = 16
HEAD_DIM_QUANTUM = 16


def _pages(tokens: int) -> int:
    return -(-tokens // PAGE_TOKENS)


def layer_slot_shape(num_kv_heads: int, head_dim: int, max_seq_len: int, attn_tp: int = 1, batch_size: int = 1,
                     sliding_window: Optional[int] = None) -> Tuple[int, ...]:
    """``(2, pages, local kv heads, 16, head_dim)`` of one owner layer on one tensor-parallel rank.  KV heads are split
    across ranks; with more ranks than heads every rank keeps one (replicated) head."""
    if head_dim % HEAD_DIM_QUANTUM:
        raise ValueError(f"head_dim {head_dim} not a multiple of {HEAD_DIM_QUANTUM}")
    if attn_tp <= 0 or (num_kv_heads % attn_tp and attn_tp % num_kv_heads):
        raise ValueError(f"{num_kv_heads} KV heads cannot be laid out over {attn_tp} ranks")
    tokens = max_seq_len if not sliding_window else min(max_seq_len, sliding_window + PAGE_TOKENS)
    return (2, batch_size * _pages(tokens), max(1, num_kv_heads // attn_tp), PAGE_TOKENS, head_dim)


def cache_plan(geom: Sequence[Any], max_seq_len: int, attn_tp: int = 1, batch_size: int = 1, *,
               bytes_per_element: int = 2, bound_sliding_layers: bool = True) -> Dict[str, Any]:
    """Plan for a geometry table (objects with ``head_dim, num_kv_heads, kv_source_layer, is_kv_shared`` and optionally
    ``sliding_window``).

    Returns ``num_layers``, ``source_map``, ``owners`` (layers that allocate), ``layers`` (per layer: ``idx, owns,
    source, head_dim, num_kv_heads, slot_shape`` - a shared layer lists its source's slot) and ``total_bytes`` over the
    owners.  Raises ``ValueError`` for a source that is out of range, itself shared, of another width, or - for a
    non-shared layer - not the layer itself."""
    n = len(geom)
    source_map = [int(g.kv_source_layer) for g in geom]
    for i, (g, src) in enumerate(zip(geom, source_map)):
        if not 0 <= src < n:
            raise ValueError(f"layer {i}: kv_source_layer {src} out of range")
        s = geom[src]
        if s.is_kv_shared:
            raise ValueError(f"layer {i}: source {src} is itself KV-shared")
        if (s.head_dim, s.num_kv_heads) != (g.head_dim, g.num_kv_heads):
            raise ValueError(f"layer {i}: source {src} geometry (hd={s.head_dim}, nkv={s.num_kv_heads}) != layer "
                             f"(hd={g.head_dim}, nkv={g.num_kv_heads})")
        if not g.is_kv_shared and src != i:
            raise ValueError(f"non-shared layer {i} must source itself, got {src}")

    def slot(layer: Any) -> Tuple[int, ...]:
        window = getattr(layer, "sliding_window", None) if bound_sliding_layers else None
        return layer_slot_shape(layer.num_kv_heads, layer.head_dim, max_seq_len, attn_tp, batch_size, window)

    layers: List[Dict[str, Any]] = [
        {"idx": i, "owns": not g.is_kv_shared, "source": src, "head_dim": int(g.head_dim),
         "num_kv_heads": int(g.num_kv_heads), "slot_shape": slot(geom[src])}
        for i, (g, src) in enumerate(zip(geom, source_map))]
    owners = [row["idx"] for row in layers if row["owns"]]
    total = 0
    for i in owners:
        count = bytes_per_element
        for d in layers[i]["slot_shape"]:
            count *= d
        total += count
    return {"num_layers": n, "source_map": source_map, "owners": owners, "layers": layers, "total_bytes": total}


def windowed_mask(offset: int, q_len: int, kv_len: int, sliding: int = 512):
    """Additive fp32 mask ``[q_len, kv_len]`` of a sliding layer (0 attend, -inf masked): the query at absolute position
    ``p = offset + row`` sees keys ``p - sliding < k <= p``.  The oracle the attention kernel's ``window`` argument is
    tested against."""
    import torch
    p = offset + torch.arange(q_len)[:, None]
    k = torch.arange(kv_len)[None, :]
    seen = (k <= p) & (k > p - sliding)
    return torch.zeros(q_len, kv_len).masked_fill(~seen, float("-inf"))


__all__ = ["cache_plan", "layer_slot_shape", "windowed_mask", "PAGE_TOKENS"]
