"""Torch-tensor front-ends of the sm_100a kernels in ``librf_b200``.

Each function checks shapes/dtypes on the host, fills the C argument block and
launches on the current CUDA stream.  There is no PyTorch fallback: if the
native library is missing these raise, so a test that passes has run the kernel.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native as N

ACT = {None: 0, "none": 0, "silu_mul": 1, "gelu_tanh_mul": 2, "gelu_tanh": 3, "gelu_erf": 4, "silu": 5}
ELT = {"add": 0, "mul": 1, "silu_mul": 2, "gelu_tanh_mul": 3, "axpy": 4, "gelu_tanh": 5, "gelu_erf": 6,
       "silu": 7, "scale": 8, "sigmoid_mul": 9, "mul_row": 10, "tanh": 11}


def dtype_code(t: torch.dtype) -> int:
    if t == torch.float16:
        return 0
    if t == torch.bfloat16:
        return 1
    raise TypeError(f"kernels take float16 or bfloat16, got {t}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


_scratch: dict = {}


def _splitk_scratch(device: torch.device, ws_bytes: int, sems: int):
    """Per-device split-K workspace + zeroed semaphores, grown on demand."""
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    ws, sem = _scratch.get(key, (None, None))
    if ws is None or ws.numel() * 4 < ws_bytes:
        ws = torch.empty(max(ws_bytes // 4, 1 << 20), dtype=torch.float32, device=device)
    if sem is None or sem.numel() < sems:
        sem = torch.zeros(max(sems, 4096), dtype=torch.int32, device=device)
    _scratch[key] = (ws, sem)
    return ws, sem


def gemm(x: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
         act: Optional[str] = None, dual: bool = False, status: Optional[torch.Tensor] = None,
         force_splits: int = 0, force_swap: int = -1, force_bn: int = 0, use_gemv: bool = False,
         ws: Optional[torch.Tensor] = None, sem: Optional[torch.Tensor] = None,
         comm=None) -> torch.Tensor:
    """``out = epilogue(x @ w.T)`` on the tcgen05 kernel (or the CUDA-core GEMV).

    ``dual=True``: ``w`` stacks ``[gate; up]`` (2N rows) and ``act`` is a ``*_mul``
    activation, giving ``act(x@gate.T) * (x@up.T)`` with N columns.
    ``w`` may be int8 with ``scale`` (per output channel) for the GEMV path.
    ``comm``: a :class:`rhinoforge_b200.parallel.symm.CommBuffers` for the fused all-reduce.
    """
    assert x.is_cuda and x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1 and w.stride(1) == 1
    M, K = x.shape
    n_rows = w.shape[0]
    assert w.shape[1] == K, (x.shape, w.shape)
    Nn = n_rows // 2 if dual else n_rows
    if out is None:
        out = torch.empty((M, Nn), dtype=x.dtype, device=x.device)
    g = N.RfGemm()
    g.x, g.ldx = x.data_ptr(), x.stride(0)
    g.w, g.ldw = w.data_ptr(), w.stride(0)
    g.out, g.ldo = out.data_ptr(), out.stride(0)
    if residual is not None:
        g.residual, g.ldr = residual.data_ptr(), residual.stride(0)
    g.bias, g.scale, g.row_scale = _ptr(bias), _ptr(scale), _ptr(row_scale)
    g.M, g.N, g.K = M, Nn, K
    g.dtype = dtype_code(x.dtype)
    g.act = ACT[act]
    g.dual_offset = Nn if dual else 0
    g.w_int8 = 1 if w.dtype == torch.int8 else 0
    g.status = _ptr(status)
    g.force_splits, g.force_swap, g.force_bn = force_splits, force_swap, force_bn
    lib = N.lib()
    if use_gemv:
        N.check(lib.rf_gemv(C.byref(g), _stream()), "rf_gemv")
        return out
    if comm is not None:
        comm.fill(g)
    need_ws, need_sem = C.c_uint64(0), C.c_int32(0)
    g.ws_bytes = 2 ** 64 - 1
    N.check(lib.rf_gemm_scratch(C.byref(g), C.byref(need_ws), C.byref(need_sem)), "rf_gemm_scratch")
    g.ws_bytes = 0
    if need_ws.value > 0:
        if ws is None or sem is None:
            ws, sem = _splitk_scratch(x.device, need_ws.value, need_sem.value)
        g.ws, g.ws_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
        g.sem, g.sem_count = sem.data_ptr(), sem.numel()
    if w.dtype == torch.int8:
        N.check(lib.rf_gemm_w8a16(C.byref(g), _stream()), "rf_gemm_w8a16")
    else:
        N.check(lib.rf_gemm(C.byref(g), _stream()), "rf_gemm")
    return out


def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, *, residual: Optional[torch.Tensor] = None,
            residual_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            gemma: bool = False, mod: Optional[torch.Tensor] = None, rows_per_mod: int = 1) -> torch.Tensor:
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    if out is None:
        out = torch.empty_like(x2)
    o2 = out.reshape(-1, H)
    N.check(N.lib().rf_rmsnorm(C.c_void_p(x2.data_ptr()), C.c_void_p(_ptr(residual)), C.c_void_p(_ptr(w)),
                               C.c_void_p(o2.data_ptr()), C.c_void_p(_ptr(residual_out)), C.c_void_p(_ptr(mod)),
                               rows_per_mod, x2.shape[0], H, C.c_int64(x2.stride(0)), C.c_int64(o2.stride(0)),
                               C.c_float(eps), 1 if gemma else 0, dtype_code(x.dtype), _stream()), "rf_rmsnorm")
    return out.reshape(x.shape)


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    if out is None:
        out = torch.empty_like(x2)
    o2 = out.reshape(-1, H)
    N.check(N.lib().rf_layernorm(C.c_void_p(x2.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(_ptr(b)),
                                 C.c_void_p(o2.data_ptr()), x2.shape[0], H, C.c_int64(x2.stride(0)),
                                 C.c_int64(o2.stride(0)), C.c_float(eps), dtype_code(x.dtype), _stream()),
            "rf_layernorm")
    return out.reshape(x.shape)


def l2norm(x: torch.Tensor, eps: float = 1e-6, out_scale: float = 1.0) -> torch.Tensor:
    H = x.shape[-1]
    x2 = x.contiguous().reshape(-1, H)
    out = torch.empty_like(x2)
    N.check(N.lib().rf_l2norm(C.c_void_p(x2.data_ptr()), C.c_void_p(out.data_ptr()), x2.shape[0], H,
                              C.c_float(eps), C.c_float(out_scale), dtype_code(x.dtype), _stream()), "rf_l2norm")
    return out.reshape(x.shape)


def gated_residual(x: torch.Tensor, y: torch.Tensor, mod: torch.Tensor, rows_per_mod: int) -> torch.Tensor:
    H = x.shape[-1]
    rows = x.numel() // H
    N.check(N.lib().rf_gated_residual(C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), C.c_void_p(mod.data_ptr()),
                                      rows_per_mod, rows, H, dtype_code(x.dtype), _stream()), "rf_gated_residual")
    return x


def qk_norm_rope_kv(qkv: torch.Tensor, Hq: int, Hkv: int, hd: int, *, pos: torch.Tensor,
                    cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                    rot_dim: Optional[int] = None, q_norm_w: Optional[torch.Tensor] = None,
                    k_norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6, gemma: bool = False,
                    axis_of_freq: Optional[torch.Tensor] = None, k_pool: Optional[torch.Tensor] = None,
                    v_pool: Optional[torch.Tensor] = None, page_table: Optional[torch.Tensor] = None,
                    seq_of_tok: Optional[torch.Tensor] = None, cache_pos: Optional[torch.Tensor] = None,
                    q_out: Optional[torch.Tensor] = None, rope_before_norm: bool = False,
                    write_k_inplace: bool = False) -> None:
    a = N.RfRopeKv()
    tokens = qkv.shape[0]
    a.qkv, a.ld = qkv.data_ptr(), qkv.stride(0)
    if q_out is not None:
        a.q_out, a.ldq = q_out.data_ptr(), q_out.stride(0)
    a.tokens, a.Hq, a.Hkv, a.hd = tokens, Hq, Hkv, hd
    a.rot_dim = hd if rot_dim is None else rot_dim
    a.q_norm_w, a.k_norm_w = _ptr(q_norm_w), _ptr(k_norm_w)
    a.eps, a.norm_mode = eps, 1 if gemma else 0
    if cos is not None:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[-1] == a.rot_dim // 2
    a.cos, a.sin = _ptr(cos), _ptr(sin)
    assert pos.dtype == torch.int32
    a.pos = pos.data_ptr()
    a.pos_stride = 1 if pos.dim() == 1 else pos.shape[1]
    if axis_of_freq is not None:
        assert axis_of_freq.dtype == torch.int8
    a.axis_of_freq = _ptr(axis_of_freq)
    a.k_pool, a.v_pool = _ptr(k_pool), _ptr(v_pool)
    if page_table is not None:
        assert page_table.dtype == torch.int32
        a.page_table, a.pt_stride = page_table.data_ptr(), page_table.stride(0)
    a.seq_of_tok, a.cache_pos = _ptr(seq_of_tok), _ptr(cache_pos)
    a.rope_before_norm, a.write_k_inplace = int(rope_before_norm), int(write_k_inplace)
    a.dtype = dtype_code(qkv.dtype)
    N.check(N.lib().rf_qk_norm_rope_kv(C.byref(a), _stream()), "rf_qk_norm_rope_kv")


def embedding(table: torch.Tensor, ids: torch.Tensor, *, out: Optional[torch.Tensor] = None, scale: float = 1.0,
              row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert ids.dtype == torch.int32
    H = table.shape[1]
    dt = row_scale.dtype if row_scale is not None else table.dtype
    if out is None:
        out = torch.empty((ids.numel(), H), dtype=dt, device=table.device)
    N.check(N.lib().rf_embedding(C.c_void_p(table.data_ptr()), C.c_void_p(ids.data_ptr()), C.c_void_p(out.data_ptr()),
                                 ids.numel(), H, C.c_int64(out.stride(0)), C.c_float(scale), dtype_code(dt),
                                 C.c_void_p(_ptr(row_scale)), _stream()), "rf_embedding")
    return out


def scatter_rows(dst: torch.Tensor, src: torch.Tensor, rows: torch.Tensor, accumulate: bool = False) -> None:
    assert rows.dtype == torch.int32
    N.check(N.lib().rf_scatter_rows(C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()), C.c_void_p(rows.data_ptr()),
                                    rows.numel(), src.shape[1], C.c_int64(dst.stride(0)), C.c_int64(src.stride(0)),
                                    int(accumulate), dtype_code(dst.dtype), _stream()), "rf_scatter_rows")


def eltwise(op: str, a: torch.Tensor, b: Optional[torch.Tensor] = None, *, alpha: float = 1.0,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty_like(a)
    period = 0
    if b is not None and b.numel() != a.numel():
        period = b.numel()
    N.check(N.lib().rf_eltwise(ELT[op], C.c_void_p(a.data_ptr()), C.c_void_p(_ptr(b)), C.c_void_p(out.data_ptr()),
                               C.c_int64(a.numel()), C.c_int64(period), C.c_float(alpha), dtype_code(a.dtype),
                               _stream()), "rf_eltwise")
    return out


def cast_u8(src: torch.Tensor, dtype: torch.dtype = torch.float16, scale: float = 1.0, shift: float = 0.0,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert src.dtype == torch.uint8
    if out is None:
        out = torch.empty(src.shape, dtype=dtype, device=src.device)
    N.check(N.lib().rf_cast_u8_f16(C.c_void_p(src.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int64(src.numel()),
                                   C.c_float(scale), C.c_float(shift), dtype_code(out.dtype), _stream()),
            "rf_cast_u8_f16")
    return out


def argmax(logits: torch.Tensor, *, offset: int = 0, return_vals: bool = False):
    rows, V = logits.shape
    lib = N.lib()
    nbytes = lib.rf_argmax_scratch_bytes(rows, V)
    scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=logits.device)
    ids = torch.empty(rows, dtype=torch.int32, device=logits.device)
    vals = torch.empty(rows, dtype=torch.float32, device=logits.device) if return_vals else None
    N.check(lib.rf_argmax(C.c_void_p(logits.data_ptr()), rows, V, C.c_int64(logits.stride(0)),
                          C.c_void_p(ids.data_ptr()), C.c_void_p(_ptr(vals)), offset, C.c_void_p(scratch.data_ptr()),
                          C.c_uint64(nbytes), dtype_code(logits.dtype), _stream()), "rf_argmax")
    return (ids, vals) if return_vals else ids


def _i32(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    assert t.dtype == torch.int32 and t.is_contiguous()
    return t.data_ptr()


def attention_prefill(q: torch.Tensor, out: torch.Tensor, *, Hq: int, Hkv: int, hd: int,
                      q_start: torch.Tensor, q_len: torch.Tensor, kv_len: torch.Tensor, max_q_len: int,
                      k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
                      page_table: Optional[torch.Tensor] = None,
                      k: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None,
                      kv_start: Optional[torch.Tensor] = None, causal: bool = True, window: int = 0,
                      mask: Optional[torch.Tensor] = None, seg_q: Optional[torch.Tensor] = None,
                      seg_k: Optional[torch.Tensor] = None, scale: float = 0.0,
                      status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Flash-style attention over ``q`` rows [tokens, Hq*hd]; KV from the paged pool or from
    contiguous ``k``/``v`` [rows, Hkv*hd] (may be column slices of a packed qkv buffer)."""
    a = N.RfAttn()
    a.q, a.ldq, a.out, a.ldo = q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0)
    a.q_rows_total = q.shape[0]
    a.num_seqs, a.Hq, a.Hkv, a.hd = q_len.numel(), Hq, Hkv, hd
    if k_pool is not None:
        a.k_pool, a.v_pool, a.pool_pages = k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0]
        a.page_table, a.pt_stride = _i32(page_table), page_table.stride(0)
    else:
        a.k, a.v, a.ldk, a.ldv, a.kv_rows_total = k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), k.shape[0]
        a.kv_start = _i32(kv_start)
    a.q_start, a.q_len, a.kv_len = _i32(q_start), _i32(q_len), _i32(kv_len)
    a.max_q_len = max_q_len
    a.causal, a.window = int(causal), window
    if mask is not None:
        assert mask.dtype in (torch.uint8, torch.bool) and mask.stride(-1) == 1
        a.mask, a.mask_ld = mask.data_ptr(), mask.stride(-2)
        a.mask_seq_stride = mask.stride(0) if mask.dim() == 3 else 0
    a.seg_q, a.seg_k = _i32(seg_q), _i32(seg_k)
    a.scale = scale
    a.status = _ptr(status)
    a.dtype = dtype_code(q.dtype)
    N.check(N.lib().rf_attn_prefill(C.byref(a), _stream()), "rf_attn_prefill")
    return out


def attention_decode(q: torch.Tensor, out: torch.Tensor, *, Hq: int, Hkv: int, hd: int, kv_len: torch.Tensor,
                     max_kv_len: int, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                     scale: float = 0.0, ws: Optional[torch.Tensor] = None,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query token per sequence against the paged KV pool (split-KV when ``ws`` is given)."""
    a = N.RfAttn()
    a.q, a.ldq, a.out, a.ldo = q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0)
    a.q_rows_total = q.shape[0]
    a.num_seqs, a.Hq, a.Hkv, a.hd = q.shape[0], Hq, Hkv, hd
    a.k_pool, a.v_pool, a.pool_pages = k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0]
    a.page_table, a.pt_stride = _i32(page_table), page_table.stride(0)
    a.kv_len = _i32(kv_len)
    a.max_kv_len = max_kv_len
    a.scale = scale
    if ws is not None:
        a.ws, a.ws_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
    a.status = _ptr(status)
    a.dtype = dtype_code(q.dtype)
    N.check(N.lib().rf_attn_decode(C.byref(a), _stream()), "rf_attn_decode")
    return out


def attn_decode_scratch(num_seqs: int, Hq: int, hd: int, device) -> torch.Tensor:
    n = N.lib().rf_attn_decode_scratch_bytes(num_seqs, Hq, hd)
    return torch.empty(n // 4, dtype=torch.float32, device=device)
