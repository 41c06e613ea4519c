"""Gemma4 host planning: per-layer geometry, signature encoding, paged KV plan with K/V sharing, window mask."""
import dataclasses
import importlib.util
import pathlib
import sys

import pytest
import torch

from rhinoforge_b200.adapters.gemma4 import (cache_plan, geometry_dyn_dims, geometry_hash, layer_geometry,
                                             layer_slot_shape, max_head_dim, max_num_kv_heads, native_layer_arrays,
                                             windowed_mask)

S, G = "sliding_attention", "full_attention"


def e4b(**over):
    cfg = dict(num_hidden_layers=12, layer_types=([S] * 5 + [G]) * 2, num_kv_shared_layers=4, head_dim=256,
               global_head_dim=512, num_attention_heads=8, num_key_value_heads=2, sliding_window=512)
    cfg.update(over)
    return cfg


def test_geometry_module_needs_nothing_but_the_standard_library():
    path = pathlib.Path(__file__).resolve().parents[1] / "rhinoforge_b200" / "adapters" / "gemma4" / "geometry.py"
    before = set(sys.modules)
    spec = importlib.util.spec_from_file_location("_gemma4_geometry_alone", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    try:
        spec.loader.exec_module(mod)
        assert not {m for m in set(sys.modules) - before if m.split(".")[0] in ("torch", "rhinoforge_b200", "numpy")}
        assert len(mod.layer_geometry(e4b())) == 12
    finally:
        del sys.modules[spec.name]


def test_layer_table_widths_and_sharing():
    geo = layer_geometry(e4b())
    assert [g.head_dim for g in geo] == ([256] * 5 + [512]) * 2
    assert [g.rope_type for g in geo[4:6]] == ["default", "proportional"]
    assert geo[0].sliding_window == 512 and geo[5].sliding_window is None
    # 12 layers, last 4 shared: owners are 0..7; sliding sharers read layer 7 (the last sliding owner), the global one layer 5
    assert [g.is_kv_shared for g in geo] == [False] * 8 + [True] * 4
    assert [g.kv_source_layer for g in geo] == [0, 1, 2, 3, 4, 5, 6, 7, 7, 7, 7, 5]
    assert all(g.has_kv_proj != g.is_kv_shared for g in geo)
    arrays = native_layer_arrays(geo)
    assert arrays["layer_type_ids"] == ([0] * 5 + [1]) * 2 and arrays["is_kv_shared"][-4:] == [1, 1, 1, 1]
    assert arrays["kv_source_layer"][-1] == 5 and set(arrays) == {"layer_type_ids", "head_dim_per_layer",
                                                                  "num_kv_heads_per_layer", "kv_source_layer",
                                                                  "is_kv_shared", "has_kv_proj"}
    assert (max_head_dim(geo), max_num_kv_heads(geo)) == (512, 2)

    class Cfg:                                                       # attribute-style configs work as well
        pass
    c = Cfg()
    c.__dict__.update(e4b(attention_k_eq_v=True, num_global_key_value_heads=4))
    alt = layer_geometry(c)
    assert alt[5].num_kv_heads == 4 and alt[0].num_kv_heads == 2
    with pytest.raises(ValueError, match="layer_types length"):
        layer_geometry(e4b(num_hidden_layers=13))
    with pytest.raises(ValueError, match="no non-shared source"):
        layer_geometry(e4b(num_kv_shared_layers=7))                  # owners 0..4 are all sliding; layer 5 is global


def _fnv1a64(values):
    h = 0xCBF29CE484222325
    for v in values:
        h ^= v & 0xFFFFFFFF
        h = (h * 0x100000001B3) % (1 << 64)
    return h % (1 << 63)


def test_signature_encoding_separates_geometries():
    geo = layer_geometry(e4b())
    flat = [v for g in geo for v in (g.head_dim, g.num_kv_heads, int(g.is_global), int(g.is_kv_shared), g.kv_source_layer)]
    assert geometry_hash(geo) == _fnv1a64(flat) and 0 <= geometry_hash(geo) < 1 << 63
    assert geometry_dyn_dims(geo) == [12, geometry_hash(geo)]
    seen = {geometry_hash(geo)}
    for change in (dict(num_kv_shared_layers=2), dict(global_head_dim=256), dict(num_key_value_heads=4),
                   dict(layer_types=[S] * 4 + [G, S] + [S] * 5 + [G])):
        h = geometry_hash(layer_geometry(e4b(**change)))
        assert h not in seen
        seen.add(h)
    assert geometry_hash(geo[::-1]) != geometry_hash(geo)            # order matters
    assert geometry_hash(layer_geometry(e4b(sliding_window=1024))) == geometry_hash(geo)   # the window is a kernel argument


def test_cache_plan_allocates_owners_only_and_bounds_sliding_layers():
    geo = layer_geometry(e4b())
    plan = cache_plan(geo, max_seq_len=8192, batch_size=2)
    assert plan["num_layers"] == 12 and plan["owners"] == list(range(8)) and plan["source_map"][8:] == [7, 7, 7, 5]
    sliding, glob = plan["layers"][0]["slot_shape"], plan["layers"][5]["slot_shape"]
    assert sliding == (2, 2 * 33, 2, 16, 256) and glob == (2, 2 * 512, 2, 16, 512)    # window 512 + one page of slack
    assert plan["layers"][11]["slot_shape"] == glob and not plan["layers"][11]["owns"] and plan["layers"][11]["source"] == 5
    want = 2 * (7 * 2 * 66 * 2 * 16 * 256 + 1 * 2 * 1024 * 2 * 16 * 512)
    assert plan["total_bytes"] == want
    dense = cache_plan(geo, max_seq_len=8192, batch_size=2, bound_sliding_layers=False)
    assert dense["layers"][0]["slot_shape"] == (2, 1024, 2, 16, 256) and dense["total_bytes"] > 3 * plan["total_bytes"]
    assert cache_plan(geo, 100)["layers"][0]["slot_shape"][1] == 7                       # shorter than the window
    assert layer_slot_shape(2, 256, 64, attn_tp=2)[2] == 1 and layer_slot_shape(2, 256, 64, attn_tp=8)[2] == 1
    with pytest.raises(ValueError, match="cannot be laid out"):
        layer_slot_shape(2, 256, 64, attn_tp=3)
    with pytest.raises(ValueError, match="multiple of 16"):
        layer_slot_shape(2, 250, 64)


def test_cache_plan_rejects_a_broken_source_map():
    geo = layer_geometry(e4b())
    swap = lambda i, **kw: [dataclasses.replace(g, **kw) if g.idx == i else g for g in geo]
    for bad, msg in ((swap(9, kv_source_layer=40), "out of range"), (swap(9, kv_source_layer=8), "itself KV-shared"),
                     (swap(9, kv_source_layer=5), "geometry"), (swap(2, kv_source_layer=1), "must source itself")):
        with pytest.raises(ValueError, match=msg):
            cache_plan(bad, 1024)


def test_windowed_mask_matches_the_definition():
    m = windowed_mask(offset=5, q_len=4, kv_len=12, sliding=3)
    assert m.shape == (4, 12) and m.dtype == torch.float32
    for q in range(4):
        for k in range(12):
            p = 5 + q
            assert (m[q, k] == 0) == (p - 3 < k <= p)
    assert torch.isinf(m[m != 0]).all() and int((m == 0).sum()) == 12
    full = windowed_mask(0, 6, 6, sliding=512)
    assert torch.equal(full == 0, torch.tril(torch.ones(6, 6, dtype=torch.bool)))
