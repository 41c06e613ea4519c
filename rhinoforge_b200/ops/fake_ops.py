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


# ----------------------------------------------------------------------------------------------- handle families
# A handle's configuration is host data, so the output shape of most ``*_forward`` ops is known without running them.
# The exception is the grid-driven vision towers: their token count is the sum over ``grid_thw`` *values*, which a
# fake tensor does not have; those refuse with a message instead of guessing.

def _handle_config(handle: int, families):
    from . import handle_ops
    return handle_ops._entry(handle, families)


def _handle_dtype(entry):
    from . import handle_ops
    return handle_ops._dtype_of(entry.config)


def _decoder_forward_meta(handle, hidden_states, *args, **kwargs):
    from . import handle_ops
    e = _handle_config(handle, handle_ops._DECODERS)
    batch = hidden_states.shape[0] if hidden_states.dim() == 3 else 1
    return hidden_states.new_empty((batch, int(e.config["vocab_size"])), dtype=_handle_dtype(e))


def _image_tower_forward_meta(family: str):
    def meta(handle, pixel_values):
        e = _handle_config(handle, (family,))
        c, B = e.config, pixel_values.shape[0]
        hidden, patch = int(c["hidden_size"]), int(c["patch_size"])
        dt = _handle_dtype(e)
        if family == "dinov3_vision":
            tokens = 1 + int(c.get("num_register_tokens", 4)) + (pixel_values.shape[2] // patch) * (pixel_values.shape[3] // patch)
            return [pixel_values.new_empty((B, tokens, hidden), dtype=dt), pixel_values.new_empty((B, hidden), dtype=dt)]
        width = hidden
        proj = getattr(e.runtime, "projector", None)
        if proj is not None:
            width = int(proj[0].shape[0])
        elif "rpu_projector_dim" in c:
            width = int(c["rpu_projector_dim"])
        return [pixel_values.new_empty((B, (int(c.get("image_size", 224)) // patch) ** 2, width), dtype=dt)]
    return meta


def _grid_tower_forward_meta(family: str):
    def meta(handle, pixel_values, grid_thw):
        from ..runtime.errors import RPUBackendError
        raise RPUBackendError(f"{family}_forward has a data-dependent output length (the sum over grid_thw); it cannot be "
                              "shape-traced with fake tensors - trace around it or pass concrete grids")
    return meta


def _pi05_forward_meta(handle, images, image_mask, tokens, token_mask, noise, num_steps=10):
    from . import handle_ops
    return torch.empty_like(noise, dtype=_handle_dtype(_handle_config(handle, handle_ops._PI05)))


def _gemma_forward_meta(handle, images, image_mask, tokens, token_mask):
    return tokens.new_empty((tokens.shape[0],), dtype=torch.int32)           # one prefix length per sequence


def _denoise_forward_meta(handle, prefix_lens, noise, num_steps=10):
    from . import handle_ops
    return torch.empty_like(noise, dtype=_handle_dtype(_handle_config(handle, handle_ops._PI05)))


def register_handle_families(lib: "torch.library.Library") -> None:
    """``Meta`` implementations of the ``<family>_forward`` ops (call after ``handle_ops.register``)."""
    from . import handle_ops
    for name in handle_ops._DECODERS:
        lib.impl(f"{name}_forward", _decoder_forward_meta, "Meta")
    for name in ("siglip", "hyvit2", "dinov3_vision"):
        lib.impl(f"{name}_forward", _image_tower_forward_meta(name), "Meta")
    for name in ("qwen3vl_vision", "qwen3_5_vision", "qwen25vl_vision"):
        lib.impl(f"{name}_forward", _grid_tower_forward_meta(name), "Meta")
    lib.impl("pi05_forward", _pi05_forward_meta, "Meta")
    lib.impl("gemma_forward", _gemma_forward_meta, "Meta")
    for name in ("adarms_forward", "pi05_denoise_step_forward", "pi05_denoise_loop_forward"):
        lib.impl(name, _denoise_forward_meta, "Meta")


__all__ = ["register", "register_handle_families"]
