"""Shape-only ("meta") implementations of the stand-alone ``torch.ops.rpu`` operators.

With these registered the operators can be traced under ``FakeTensorMode`` / on ``device="meta"`` (shape propagation,
export, memory planning) without touching a GPU: a fake CUDA tensor has no data pointer, so the real implementations,
which hand pointers to the native library, cannot run there.  The reference keeps the same kind of shims in
``python/rpu_backend/graph/fake_dispatch.py``.  Only output shapes, dtypes and devices are produced here.
"""
from __future__ import annotations


import torch


def _rms_norm(x, weight, eps):
    return torch.empty_like(x)


def _apply_rotary_pos_emb(x, cos, sin, positions):
    return torch.empty_like(x)


def _sdpa_unified(q, k, v, is_causal=False, scale=0.0):
    return torch.empty_like(q)


def _gather_embedding(table, ids):
    return table.new_empty((*ids.shape, table.shape[1]))


def _assemble_inputs_embeds(text, vision, rows):
    return torch.empty_like(text)


def _assemble_inputs_embeds_rev(embeds, rows):
    return embeds.new_empty((rows.numel(), embeds.shape[1]))


def _cast_uint8_fp16(x, scale=1.0, shift=0.0):
    return x.new_empty(x.shape, dtype=torch.float16)


def _conv2d_mc_nhwc(x, weight, bias, stride=1, padding=0):
    B, H, W, _ = x.shape
    O, _, kh, kw = weight.shape
    return x.new_empty((B, (H + 2 * padding - kh) // stride + 1, (W + 2 * padding - kw) // stride + 1, O))


def _lm_head_logits_top1(hidden, weight):
    return hidden.new_empty((hidden.shape[0],), dtype=torch.int32)


def _argmax_lastdim_host(x):
    return x.new_empty(x.shape[:-1], dtype=torch.int32)


def _moe_select(logits, bias, k, scale=1.0):
    T = logits.shape[0]
    return logits.new_empty((T, k), dtype=torch.int32), logits.new_empty((T, k), dtype=torch.float32)


_META = {
    "rms_norm": _rms_norm, "apply_rotary_pos_emb": _apply_rotary_pos_emb,
    "scaled_dot_product_attention_unified": _sdpa_unified, "gather_embedding": _gather_embedding,
    "assemble_inputs_embeds": _assemble_inputs_embeds, "assemble_inputs_embeds_rev": _assemble_inputs_embeds_rev,
    "cast_uint8_fp16": _cast_uint8_fp16, "conv2d_mc_nhwc": _conv2d_mc_nhwc, "lm_head_logits_top1": _lm_head_logits_top1,
    "argmax_lastdim_host": _argmax_lastdim_host, "moe_select": _moe_select,
}


def register(lib: "torch.library.Library") -> None:
    """Attach the shape-only implementations to the ``Meta`` dispatch key of ``lib`` (the ``rpu`` namespace)."""
    for name, fn in _META.items():
        lib.impl(name, fn, "Meta")


__all__ = ["register"]
