"""``torch.ops.rpu.*``: the stand-alone operator surface, registered through ``torch.library``.

Every op takes and returns ordinary CUDA tensors and dispatches to the hand-written kernels of
:mod:`rhinoforge_b200.ops.kernels`; there is no eager PyTorch fallback on a GPU box (CPU tensors get a
plain PyTorch implementation so that host-only tooling and tests can call the same names).  Names and
argument order follow the reference's schema list (``src/core/rpu_dispatch_registrations.inc:5-852``):
``rms_norm``, ``apply_rotary_pos_emb``, ``scaled_dot_product_attention_unified`` (layout ``[B, S, H, D]``),
``gather_embedding``, ``assemble_inputs_embeds``, ``cast_uint8_fp16``, ``linear_into``,
``assemble_inputs_embeds_rev``, ``cast_uint8_fp16_into``, ``conv2d_mc_nhwc``, ``lm_head_logits_top1``,
``argmax_lastdim_host``, ``moe_select``, ``reset_graph_cache`` and the ``spm_alloc_*`` controls (the scratch-pad
planner they steer does not exist on this hardware: they report the activation-arena figures instead).
The model handle families (``causal_decoder_*`` ...) are registered by :mod:`rhinoforge_b200.ops.handle_ops`.
"""
from __future__ import annotations

from typing import Optional

import torch

_LIB = None


def _k():
    from . import kernels
    return kernels


def _rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if not x.is_cuda:
        xf = x.float()
        return (weight.float() * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps))).to(x.dtype)
    shape = x.shape
    return _k().rmsnorm(x.reshape(-1, shape[-1]).contiguous(), weight, eps).view(shape)


def _apply_rotary_pos_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on ``x [tokens, heads, head_dim]`` with tables ``[max_pos, head_dim/2]`` (fp32) and int32 positions."""
    T, H, D = x.shape
    if not x.is_cuda:
        c, s = cos[positions.long()][:, None].float(), sin[positions.long()][:, None].float()
        c, s = torch.cat((c, c), -1), torch.cat((s, s), -1)
        xf = x.float()
        rot = torch.cat((-xf[..., D // 2:], xf[..., :D // 2]), -1)
        return (xf * c + rot * s).to(x.dtype)
    buf = x.reshape(T, H * D).clone()
    _k().qk_norm_rope_kv(buf, H, 0, D, pos=positions.to(torch.int32).contiguous(), cos=cos, sin=sin, write_k_inplace=True)
    return buf.view(T, H, D)


def _sdpa_unified(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False, scale: float = 0.0) -> torch.Tensor:
    """``q [B, Sq, Hq, D]``, ``k``/``v`` ``[B, Sk, Hkv, D]`` -> ``[B, Sq, Hq, D]`` (the unified layout)."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    if not q.is_cuda:
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                             is_causal=is_causal, scale=scale or None, enable_gqa=Hq != Hkv)
        return o.transpose(1, 2).contiguous()
    K = _k()
    q2, k2, v2 = q.reshape(B * Sq, Hq * D), k.reshape(B * Sk, Hkv * D), v.reshape(B * Sk, Hkv * D)
    out = torch.empty_like(q2)
    i32 = dict(dtype=torch.int32, device=q.device)
    qs, ks = torch.arange(B, **i32) * Sq, torch.arange(B, **i32) * Sk
    K.attention_prefill(q2.contiguous(), out, Hq=Hq, Hkv=Hkv, hd=D, q_start=qs.contiguous(), q_len=torch.full((B,), Sq, **i32),
                        kv_len=torch.full((B,), Sk, **i32), max_q_len=Sq, k=k2.contiguous(), v=v2.contiguous(),
                        kv_start=ks.contiguous(), causal=is_causal, scale=scale)
    return out.view(B, Sq, Hq, D)


def _gather_embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    if not table.is_cuda:
        return torch.nn.functional.embedding(ids.long(), table)
    return _k().embedding(table, ids.reshape(-1).to(torch.int32).contiguous()).view(*ids.shape, table.shape[1])


def _assemble_inputs_embeds(text: torch.Tensor, vision: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """Copy of ``text [T, H]`` whose rows ``rows[i]`` are replaced by ``vision[i]`` (image-placeholder splice)."""
    out = text.clone()
    if not text.is_cuda:
        out[rows.long()] = vision.to(out.dtype)
        return out
    _k().scatter_rows(out, vision.to(out.dtype).contiguous(), rows.to(torch.int32).contiguous())
    return out


def _assemble_inputs_embeds_rev(embeds: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """The inverse gather: rows ``rows[i]`` of ``embeds [T, H]`` as a ``[len(rows), H]`` tensor (vision rows read back)."""
    if not embeds.is_cuda:
        return embeds[rows.long()].clone()
    return _k().embedding(embeds.contiguous(), rows.reshape(-1).to(torch.int32).contiguous())


def _cast_uint8_fp16_into(x: torch.Tensor, out: torch.Tensor, scale: float = 1.0, shift: float = 0.0) -> torch.Tensor:
    out.copy_(_cast_uint8_fp16(x, scale, shift).view_as(out))
    return out


def _conv2d_mc_nhwc(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], stride: int = 1,
                    padding: int = 0) -> torch.Tensor:
    """``x [B, H, W, C]`` (channels last) with ``weight [O, C, kh, kw]`` -> ``[B, H', W', O]``.  A non-overlapping
    convolution (stride == kernel, no padding: every patch embedding) is one GEMM over the patch matrix; other
    geometries are off the hot path and go to the framework's convolution."""
    O, Cc, kh, kw = weight.shape
    B, Hh, Ww, _ = x.shape
    if x.is_cuda and stride == kh == kw and padding == 0 and Hh % kh == 0 and Ww % kw == 0 and (Cc * kh * kw) % 8 == 0:
        gh, gw = Hh // kh, Ww // kw
        cols = x.reshape(B, gh, kh, gw, kw, Cc).permute(0, 1, 3, 5, 2, 4).reshape(B * gh * gw, Cc * kh * kw).contiguous()
        y = _k().gemm(cols, weight.reshape(O, -1).to(x.dtype).contiguous(), bias=None if bias is None else bias.to(x.dtype))
        return y.view(B, gh, gw, O)
    y = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2), weight.to(x.dtype), None if bias is None else bias.to(x.dtype),
                                   stride=stride, padding=padding)
    return y.permute(0, 2, 3, 1).contiguous()


_SPM = {"initialised": False, "temporary_resets": 0, "full_resets": 0}


def _spm_alloc_init() -> None:
    _SPM["initialised"] = True


def _spm_alloc_reset_temporary() -> None:
    _SPM["temporary_resets"] += 1


def _spm_alloc_reset_all() -> None:
    _SPM["full_resets"] += 1


def _spm_alloc_dump() -> str:
    """One line of allocator state.  There is no scratch-pad planner here: activations live in one arena per native
    handle, sized at creation, and the caching allocator owns device memory."""
    import json
    dev = {}
    if torch.cuda.is_available():
        dev = {"allocated_bytes": int(torch.cuda.memory_allocated()), "reserved_bytes": int(torch.cuda.memory_reserved())}
    return json.dumps({**_SPM, **dev})


def _cast_uint8_fp16(x: torch.Tensor, scale: float = 1.0, shift: float = 0.0) -> torch.Tensor:
    if not x.is_cuda:
        return (x.float() * scale + shift).half()
    return _k().cast_u8(x.contiguous(), torch.float16, scale, shift)


def _linear_into(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        out.copy_(torch.nn.functional.linear(x, weight, bias))
        return out
    _k().gemm(x.reshape(-1, x.shape[-1]).contiguous(), weight, bias=bias, out=out.view(-1, weight.shape[0]))
    return out


def _lm_head_logits_top1(hidden: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Greedy token ids ``[rows]`` of ``hidden [rows, H] @ weight[V, H]^T`` (GEMM + two-stage arg-max on the device)."""
    if not hidden.is_cuda:
        return (hidden.float() @ weight.float().t()).argmax(-1).to(torch.int32)
    K = _k()
    return K.argmax(K.gemm(hidden.contiguous(), weight))


def _argmax_lastdim_host(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return x.float().argmax(-1).to(torch.int32)
    return _k().argmax(x.reshape(-1, x.shape[-1]).contiguous()).view(x.shape[:-1])


def _moe_select(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, scale: float = 1.0):
    if not logits.is_cuda:
        sc = torch.sigmoid(logits.float())
        key = sc + (bias.float() if bias is not None else 0.0)
        idx = torch.sort(key, dim=-1, descending=True, stable=True).indices[:, :k]
        w = torch.gather(sc, 1, idx)
        return idx.to(torch.int32), w / w.sum(-1, keepdim=True) * scale
    ids, w = _k().moe_select(logits.contiguous(), k, bias=bias, scale=scale)
    return ids, w


def register() -> bool:
    """Define the ``rpu`` operator namespace once; returns False when it already exists (re-import)."""
    global _LIB
    if _LIB is not None:
        return False
    try:
        lib = torch.library.Library("rpu", "DEF")
    except RuntimeError:
        return False
    defs = (
        ("rms_norm(Tensor x, Tensor weight, float eps) -> Tensor", _rms_norm),
        ("apply_rotary_pos_emb(Tensor x, Tensor cos, Tensor sin, Tensor positions) -> Tensor", _apply_rotary_pos_emb),
        ("scaled_dot_product_attention_unified(Tensor q, Tensor k, Tensor v, bool is_causal=False, float scale=0.0) -> Tensor",
         _sdpa_unified),
        ("gather_embedding(Tensor table, Tensor ids) -> Tensor", _gather_embedding),
        ("assemble_inputs_embeds(Tensor text, Tensor vision, Tensor rows) -> Tensor", _assemble_inputs_embeds),
        ("cast_uint8_fp16(Tensor x, float scale=1.0, float shift=0.0) -> Tensor", _cast_uint8_fp16),
        ("assemble_inputs_embeds_rev(Tensor embeds, Tensor rows) -> Tensor", _assemble_inputs_embeds_rev),
        ("cast_uint8_fp16_into(Tensor x, Tensor(a!) out, float scale=1.0, float shift=0.0) -> Tensor(a!)", _cast_uint8_fp16_into),
        ("conv2d_mc_nhwc(Tensor x, Tensor weight, Tensor? bias, int stride=1, int padding=0) -> Tensor", _conv2d_mc_nhwc),
        ("spm_alloc_init() -> ()", _spm_alloc_init),
        ("spm_alloc_reset_temporary() -> ()", _spm_alloc_reset_temporary),
        ("spm_alloc_reset_all() -> ()", _spm_alloc_reset_all),
        ("spm_alloc_dump() -> str", _spm_alloc_dump),
        ("linear_into(Tensor x, Tensor weight, Tensor? bias, Tensor(a!) out) -> Tensor(a!)", _linear_into),
        ("lm_head_logits_top1(Tensor hidden, Tensor weight) -> Tensor", _lm_head_logits_top1),
        ("argmax_lastdim_host(Tensor x) -> Tensor", _argmax_lastdim_host),
        ("moe_select(Tensor logits, Tensor? bias, int k, float scale=1.0) -> (Tensor, Tensor)", _moe_select),
    )
    for schema, fn in defs:
        lib.define(schema)
        lib.impl(schema.split("(")[0], fn, "CompositeExplicitAutograd")
    lib.define("reset_graph_cache() -> ()")

    def _reset():
        from ..graph import reset_graph_cache
        reset_graph_cache()
    lib.impl("reset_graph_cache", _reset, "CompositeExplicitAutograd")
    from . import fake_ops, handle_ops
    fake_ops.register(lib)
    handle_ops.register(lib)
    fake_ops.register_handle_families(lib)
    _LIB = lib
    return True


__all__ = ["register"]
