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


GEMM_PLAN_KEYS = ("swap", "bn", "splits", "stages", "grid_x", "grid_y", "smem", "k_blocks", "persistent", "two_shot")


def gemm_plan(M: int, N_out: int, K: int, *, dtype: torch.dtype = torch.float16, dual: bool = False, packed: bool = True,
              int8: bool = False, force_splits: int = 0) -> Optional[dict]:
    """The launch plan the library would pick for ``[M, K] x [N_out, K]^T`` - swap-AB, tile width, K splits, ring stages,
    grid, shared memory, persistent / two-shot form.  A host-side query (no device, no launch); ``None`` when the native
    library is not built."""
    if not N.available():
        return None
    g = N.RfGemm()
    g.M, g.N, g.K, g.dtype, g.force_swap, g.force_splits = M, N_out, K, 0 if dtype == torch.float16 else 1, -1, force_splits
    g.w_packed = int(packed)
    g.x = g.w = g.out = 4096                                  # placeholders: the planner checks alignment only
    g.ldx, g.ldw, g.ldo = K, K, N_out
    if dual:
        g.dual_offset, g.act = N_out, 1
    if int8:
        g.w_int8, g.scale = 1, 4096
    out = (C.c_int32 * len(GEMM_PLAN_KEYS))()
    if N.lib().rf_gemm_plan_info(C.byref(g), out) != 0:
        return None
    return dict(zip(GEMM_PLAN_KEYS, (int(v) for v in out)))


def gemm(x: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
         act: Optional[str] = None, dual: bool = False, status: Optional[torch.Tensor] = None,
         force_splits: int = 0, force_swap: int = -1, force_bn: int = 0, use_gemv: bool = False,
         ws: Optional[torch.Tensor] = None, sem: Optional[torch.Tensor] = None,
         comm=None, packed_shape: Optional[tuple] = None, w_scratch: Optional[torch.Tensor] = None,
         publish: bool = False, norm_w: Optional[torch.Tensor] = None, norm_out: Optional[torch.Tensor] = None,
         norm_eps: float = 1e-6, norm_gemma: bool = False, w_bits: int = 0, w_group: int = 0,
         w_fp4: bool = False, ss_out: Optional[torch.Tensor] = None, ss_in: Optional[torch.Tensor] = None,
         ss_dim: int = 0, ss_eps: float = 1e-6) -> torch.Tensor:
    """``out = epilogue(x @ w.T)`` on the tcgen05 kernel (or the CUDA-core GEMV).

    ``dual=True``: ``w`` stacks ``[gate; up]`` (2N rows) and ``act`` is a ``*_mul``
    activation, giving ``act(x@gate.T) * (x@up.T)`` with N columns.
    ``w`` may be int8 with ``scale`` (per output channel) for the GEMV path.
    ``comm``: a :class:`rhinoforge_b200.parallel.symm.CommBuffers` for the fused all-reduce.
    ``w_scratch``: device bytes (twice the packed int8 image) that let a W8A16 GEMM of more than 256 tokens widen the
    weights once and run the 16-bit kernels.
    ``publish`` (with ``comm``, at most 256 rows): the GEMM only pushes its partial rows to the peers and exits;
    ``rf_ar_consume`` then waits, reduces, adds ``residual`` and, with ``norm_w`` / ``norm_out``, writes the RMSNorm of
    the finished rows (``norm_gemma``: ``(1 + w)`` weights).
    ``w_bits=4``: ``w`` is the int4 image made by :func:`pack_weight_int4` (``packed_shape`` required); ``w_group`` is
    its scale group (0: per-channel ``scale`` vector, else 32 / 64 / 128 with the scales inside the image).
    ``w_fp4``: the nibbles are e2m1 codes (:func:`pack_weight_nvfp4`, scale group 16).
    ``ss_out`` (fp32 ``[ceil(N / 128), ld >= M]``, at most 256 rows): also receives the sum of squares of the finished
    output values per 128-column tile and token.  ``ss_in`` (the ``ss_out`` of the GEMM that produced ``x``): the result
    is scaled per token by ``rsqrt(sum(ss_in[:, token]) / ss_dim + ss_eps)``: an RMSNorm of ``x`` whose weights were
    multiplied into the columns of ``w`` beforehand.
    """
    M, K = x.shape
    if packed_shape is not None:          # ``w`` is the tile-major image made by pack_weight(); (rows, K) is its logical shape
        n_rows, wk = packed_shape
        assert wk == K and x.is_cuda and x.stride(1) == 1
    else:
        assert x.is_cuda and x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1 and w.stride(1) == 1
        n_rows = w.shape[0]
        assert w.shape[1] == K, (x.shape, w.shape)
    Nn = n_rows // 2 if dual else n_rows
    if out is None:
        out = torch.empty((M, Nn), dtype=x.dtype, device=x.device)
    g = N.RfGemm()
    g.x, g.ldx = x.data_ptr(), x.stride(0)
    g.w, g.ldw = w.data_ptr(), (K if packed_shape is not None else w.stride(0))
    g.w_packed = 1 if packed_shape is not None else 0
    g.out, g.ldo = out.data_ptr(), out.stride(0)
    if residual is not None:
        g.residual, g.ldr = residual.data_ptr(), residual.stride(0)
    g.bias, g.scale, g.row_scale = _ptr(bias), _ptr(scale), _ptr(row_scale)
    g.M, g.N, g.K = M, Nn, K
    g.dtype = dtype_code(x.dtype)
    g.act = ACT[act]
    g.dual_offset = Nn if dual else 0
    g.w_int8 = 1 if (w.dtype == torch.int8 or w_bits == 4) else 0
    if w_bits == 4:
        if packed_shape is None or w.dtype != torch.uint8:
            raise ValueError("w_bits=4 takes the uint8 image made by pack_weight_int4 together with packed_shape")
        g.w_bits, g.w_group, g.w_fp4 = 4, w_group, int(w_fp4)
    g.status = _ptr(status)
    for t in (ss_out, ss_in):
        if t is not None:
            assert t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1 and t.is_cuda
            g.ss_ld = t.stride(0)
    if ss_out is not None:
        assert ss_out.shape[0] >= (Nn + 127) // 128
        g.ss_out = ss_out.data_ptr()
    if ss_in is not None:
        g.ss_in, g.ss_tiles, g.ss_dim, g.ss_eps = ss_in.data_ptr(), ss_in.shape[0], ss_dim or K, ss_eps
    g.force_splits, g.force_swap, g.force_bn = force_splits, force_swap, force_bn
    if w_scratch is not None:
        g.w_scratch, g.w_scratch_bytes = w_scratch.data_ptr(), w_scratch.numel() * w_scratch.element_size()
    lib = N.lib()
    if use_gemv:
        N.check(lib.rf_gemv(C.byref(g), _stream()), "rf_gemv")
        return out
    if comm is not None:
        comm.fill(g)
    if publish:
        if comm is None:
            raise ValueError("publish=True needs comm buffers")
        g.ar_publish = 1
        ctas = lib.rf_gemm_grid_ctas(C.byref(g))
        if ctas <= 0:
            N.check(ctas, "rf_gemm_grid_ctas")
    need_ws, need_sem = C.c_uint64(0), C.c_int32(0)
    g.ws_bytes = 2 ** 64 - 1
    N.check(lib.rf_gemm_scratch(C.byref(g), C.byref(need_ws), C.byref(need_sem)), "rf_gemm_scratch")
    g.ws_bytes = 0
    if need_ws.value > 0:
        if ws is None or sem is None:
            ws, sem = _splitk_scratch(x.device, need_ws.value, need_sem.value)
        g.ws, g.ws_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
        g.sem, g.sem_count = sem.data_ptr(), sem.numel()
    if w_bits == 4:
        N.check(lib.rf_gemm_w4a16(C.byref(g), _stream()), "rf_gemm_w4a16")
    elif w.dtype == torch.int8:
        N.check(lib.rf_gemm_w8a16(C.byref(g), _stream()), "rf_gemm_w8a16")
    else:
        N.check(lib.rf_gemm(C.byref(g), _stream()), "rf_gemm")
    if publish:
        a = comm.consume_args(M, Nn, ctas, out, residual=residual, norm_w=norm_w, norm_out=norm_out, eps=norm_eps,
                              norm_mode=0 if norm_w is None else (2 if norm_gemma else 1), status=status)
        N.check(lib.rf_ar_consume(C.byref(a), _stream()), "rf_ar_consume")
    return out


def pack_weight(w: torch.Tensor, sections: int = 1) -> torch.Tensor:
    """Tile-major image of a row-major ``[rows, K]`` weight (16-bit or int8) for ``gemm(..., packed_shape=)``.

    Blocks of 128 rows x 64 columns are stored contiguously, ordered ``[row tile][k block]``; a 16-bit
    block is the 128-byte-swizzled shared-memory image (16-byte chunk ``c`` of row ``r`` sits at chunk
    ``c ^ (r % 8)``), an int8 block is plain row-major.  ``sections`` > 1 (GLU gate/up stacks) pads every
    section to a multiple of 128 rows.  Rows/columns beyond the logical shape are zero."""
    rows, Kd = w.shape
    assert rows % sections == 0
    per = rows // sections
    rt, kb = (per + 127) // 128, (Kd + 63) // 64
    out = torch.zeros((sections, rt * 128, kb * 64), dtype=w.dtype, device=w.device)
    out[:, :per, :Kd] = w.view(sections, per, Kd)
    out = out.view(sections * rt, 128, kb, 64).permute(0, 2, 1, 3).contiguous()        # [tile, kb, 128, 64]
    if w.element_size() == 2:
        blk = out.view(sections * rt, kb, 128, 8, 8)                                    # 8 chunks of 8 elements
        r = torch.arange(128, device=w.device)[:, None]
        c = torch.arange(8, device=w.device)[None, :]
        src = (c ^ (r % 8)).view(1, 1, 128, 8, 1).expand_as(blk)                        # position p holds chunk p ^ (r%8)
        out = torch.gather(blk, 3, src).contiguous()
    return out.view(-1)


_W4_NIBBLE_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)       # nibble j of a 32-bit word holds this column of its group of eight


def pack_weight_int4(q: torch.Tensor, scales: Optional[torch.Tensor] = None, group: int = 0, *, sections: int = 1,
                     dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Tile-major int4 image of ``q`` (``[rows, K]`` int8 values in ``[-8, 7]``) for ``gemm(..., w_bits=4)``.

    Blocks of 128 rows x 64 columns are contiguous, ordered ``[row tile][k block]``.  A block is 4096 bytes of nibbles
    (row-major, two's complement; inside every group of eight columns the nibbles are stored in the order
    0, 2, 4, 6, 1, 3, 5, 7, so that one shift-and-mask yields pairs of neighbouring columns) followed, for
    ``group`` in (32, 64, 128), by the block's ``128 x (64 / min(group, 64))`` scales in ``dtype`` taken from
    ``scales [rows, K / group]``.  ``group=0``: no scales in the image (one scale per output channel goes to the GEMM's
    ``scale`` argument).  Padding rows / columns are zero nibbles with scale 0."""
    rows, Kd = q.shape
    assert rows % sections == 0 and group in (0, 16, 32, 64, 128) and (group == 0 or Kd % group == 0)
    per = rows // sections
    rt, kb = (per + 127) // 128, (Kd + 63) // 64
    dev = q.device
    full = torch.zeros((sections, rt * 128, kb * 64), dtype=torch.int16, device=dev)
    full[:, :per, :Kd] = (q.view(sections, per, Kd).to(torch.int16) & 0xF)
    blk = full.view(sections * rt, 128, kb, 8, 8).permute(0, 2, 1, 3, 4)                   # [tile, kb, 128, 8 groups, 8]
    blk = blk[..., list(_W4_NIBBLE_ORDER)]                                                # storage order of the nibbles
    byts = (blk[..., 0::2] | (blk[..., 1::2] << 4)).to(torch.uint8).reshape(sections * rt, kb, 128 * 32)
    if group == 0:
        return byts.reshape(-1).contiguous()
    assert scales is not None and tuple(scales.shape) == (rows, Kd // group)
    ge = min(group, 64)
    ns = 64 // ge
    sc = torch.zeros((sections, rt * 128, kb * ns), dtype=dtype, device=dev)
    col = (torch.arange(kb * ns, device=dev) * ge) // group                               # scale column of every (kb, sub-group)
    valid = col < Kd // group
    sc[:, :per, valid] = scales.to(dev, dtype).view(sections, per, -1)[:, :, col[valid]]
    sc = sc.view(sections * rt, 128, kb, ns).permute(0, 2, 1, 3).contiguous().view(sections * rt, kb, 128 * ns)
    img = torch.cat((byts, sc.view(torch.uint8).view(sections * rt, kb, -1)), -1)
    return img.reshape(-1).contiguous()


def pack_weight_nvfp4(codes: torch.Tensor, scale_codes_gn: torch.Tensor, tensor_scale, *, sections: int = 1,
                      dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Tile-major image of an NVFP4 weight for ``gemm(..., w_bits=4, w_group=16, w_fp4=True)``: ``codes [rows, K]`` e2m1
    codes, ``scale_codes_gn [K / 16, rows]`` e4m3 block scales (as bytes) and the fp32 tensor scale, as
    ``quant.nvfp4_pack.quantize_nvfp4`` returns them.  The two scale levels are multiplied out into one ``dtype`` scale
    per 16 columns, stored inside the image like the int4 group scales."""
    eff = scale_codes_gn.t().contiguous().view(torch.float8_e4m3fn).float() * float(tensor_scale)
    return pack_weight_int4(codes, eff, 16, sections=sections, dtype=dtype)


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
                    write_k_inplace: bool = False, v_norm: bool = False) -> None:
    """Per-head RMSNorm and rotary embedding of the q / k heads of a packed ``[tokens, (Hq + 2 Hkv) * hd]`` buffer (in place
    when no pool is given), K / V insertion into a paged pool when one is.  ``v_norm``: every value head also gets an
    unweighted RMSNorm in place."""
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
    a.v_norm = int(v_norm)
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
                      status: Optional[torch.Tensor] = None, max_kv_len: int = 0) -> torch.Tensor:
    """Flash-style attention over ``q`` rows [tokens, Hq*hd]; KV from the paged pool or from
    contiguous ``k``/``v`` [rows, Hkv*hd] (may be column slices of a packed qkv buffer).
    ``max_kv_len``: a host-side bound on ``kv_len`` (0: unknown); short contiguous problems (at most 64 query rows per
    sequence over at most 512 keys, heads of 64 / 128, causal / window masks only) then take the low-latency kernel."""
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
    a.max_kv_len = int(max_kv_len)
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


# ----------------------------------------------------------------------------- linear attention (GDN)
def causal_conv1d(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, *, q_start: Optional[torch.Tensor] = None,
                  q_len: Optional[torch.Tensor] = None, max_q_len: int = 1, slot: Optional[torch.Tensor] = None,
                  num_seqs: Optional[int] = None, silu: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Depthwise causal conv (kernel 4) + SiLU over packed rows ``x [T, >=C]`` (pitch = ``x.stride(0)``) with the
    carried ``state [slots, K-1, C]`` (updated in place).  Without ``q_start``/``q_len``: one token per sequence."""
    Cc, Kw = w.shape
    a = N.RfConv1d()
    if out is None:
        out = torch.empty((x.shape[0], Cc), dtype=x.dtype, device=x.device)
    a.x, a.ldx, a.y, a.ldy = x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0)
    a.w, a.state = w.data_ptr(), state.data_ptr()
    a.q_start, a.q_len, a.slot = _i32(q_start), _i32(q_len), _i32(slot)
    a.num_seqs = int(num_seqs if num_seqs is not None else (q_len.numel() if q_len is not None else x.shape[0]))
    a.max_q_len, a.C, a.K, a.silu, a.dtype = max_q_len, Cc, Kw, int(silu), dtype_code(x.dtype)
    N.check(N.lib().rf_causal_conv1d(C.byref(a), _stream()), "rf_causal_conv1d")
    return out


def gdn_recurrent(qkv: torch.Tensor, b: torch.Tensor, a_: torch.Tensor, state: torch.Tensor, A_log: torch.Tensor,
                  dt_bias: torch.Tensor, *, Hk: int, Hv: int, Dk: int, Dv: int, q_start: Optional[torch.Tensor] = None,
                  q_len: Optional[torch.Tensor] = None, slot: Optional[torch.Tensor] = None,
                  fresh: Optional[torch.Tensor] = None, num_seqs: Optional[int] = None,
                  out: Optional[torch.Tensor] = None, chunked: bool = False) -> torch.Tensor:
    """Gated delta rule; ``qkv [T, 2*Hk*Dk + Hv*Dv]``, ``b``/``a_`` ``[T, >=Hv]`` views with a common pitch,
    ``state`` fp32 ``[slots, Hv, Dk, Dv]`` (updated in place).  Returns ``[T, Hv*Dv]``.  ``chunked``: the block-parallel
    form (64 tokens per step on the tensor cores) instead of the token-by-token kernel; same contract."""
    assert state.dtype == torch.float32 and A_log.dtype == torch.float32 and dt_bias.dtype == torch.float32
    assert b.stride(0) == a_.stride(0)
    g = N.RfGdn()
    if out is None:
        out = torch.empty((qkv.shape[0], Hv * Dv), dtype=qkv.dtype, device=qkv.device)
    g.qkv, g.ld = qkv.data_ptr(), qkv.stride(0)
    g.b, g.a, g.ld_ba = b.data_ptr(), a_.data_ptr(), b.stride(0)
    g.out, g.ldo, g.state = out.data_ptr(), out.stride(0), state.data_ptr()
    g.A_log, g.dt_bias = A_log.data_ptr(), dt_bias.data_ptr()
    g.q_start, g.q_len, g.slot, g.fresh = _i32(q_start), _i32(q_len), _i32(slot), _i32(fresh)
    g.num_seqs = int(num_seqs if num_seqs is not None else (q_len.numel() if q_len is not None else qkv.shape[0]))
    g.Hk, g.Hv, g.Dk, g.Dv, g.dtype = Hk, Hv, Dk, Dv, dtype_code(qkv.dtype)
    if chunked:
        N.check(N.lib().rf_gdn_chunked(C.byref(g), _stream()), "rf_gdn_chunked")
    else:
        N.check(N.lib().rf_gdn_recurrent(C.byref(g), _stream()), "rf_gdn_recurrent")
    return out


def rmsnorm_gated(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, heads: int, eps: float,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``(w * rmsnorm(x[t, h, :])) * silu(z[t, h, :])`` with ``x``/``z`` ``[T, heads*D]`` row views."""
    D = w.numel()
    if out is None:
        out = torch.empty((x.shape[0], heads * D), dtype=x.dtype, device=x.device)
    N.check(N.lib().rf_rmsnorm_gated(C.c_void_p(x.data_ptr()), C.c_int64(x.stride(0)), C.c_void_p(z.data_ptr()),
                                     C.c_int64(z.stride(0)), C.c_void_p(w.data_ptr()), C.c_void_p(out.data_ptr()),
                                     C.c_int64(out.stride(0)), x.shape[0], heads, D, C.c_float(eps), dtype_code(x.dtype),
                                     _stream()), "rf_rmsnorm_gated")
    return out


def sigmoid_gate(a: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """In place ``a *= sigmoid(g)``; both ``[T, C]`` row views (pitches may differ)."""
    N.check(N.lib().rf_sigmoid_gate(C.c_void_p(a.data_ptr()), C.c_int64(a.stride(0)), C.c_void_p(g.data_ptr()),
                                    C.c_int64(g.stride(0)), a.shape[0], a.shape[1], dtype_code(a.dtype), _stream()),
            "rf_sigmoid_gate")
    return a


def cumsum(x: torch.Tensor) -> torch.Tensor:
    """Inclusive cumulative sum over the last dim (fp32, contiguous)."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    y = torch.empty_like(x)
    n = x.shape[-1]
    N.check(N.lib().rf_cumsum_f32(C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), x.numel() // n, n, _stream()),
            "rf_cumsum_f32")
    return y


def unit_tril_inv(m: torch.Tensor) -> torch.Tensor:
    """``(I - tril(m, -1))^-1`` for a batch of ``[n, n]`` fp32 blocks, ``n <= 64``."""
    assert m.dtype == torch.float32 and m.is_contiguous() and m.shape[-1] == m.shape[-2]
    out = torch.empty_like(m)
    n = m.shape[-1]
    N.check(N.lib().rf_unit_tril_inv_f32(C.c_void_p(m.data_ptr()), C.c_void_p(out.data_ptr()), m.numel() // (n * n), n,
                                         _stream()), "rf_unit_tril_inv_f32")
    return out


# ----------------------------------------------------------------------------- mixture of experts
def moe_select(logits: torch.Tensor, k: int, *, bias: Optional[torch.Tensor] = None, score_fn: str = "sigmoid",
               norm_topk: bool = True, scale: float = 1.0, dense: bool = False):
    """Router top-k.  Returns ``(ids [T,k] int32, weights [T,k] fp32)`` and, with ``dense=True``, also the
    ``[T, E]`` matrix of routing weights (zero for unselected experts) in the logits' dtype."""
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    dw = torch.empty((T, E), dtype=logits.dtype, device=logits.device) if dense else None
    if bias is not None:
        assert bias.dtype == torch.float32
    N.check(N.lib().rf_moe_select(C.c_void_p(logits.data_ptr()), C.c_int64(logits.stride(0)), C.c_void_p(_ptr(bias)), T, E, k,
                                  {"sigmoid": 0, "softmax": 1}[score_fn], int(norm_topk), C.c_float(scale),
                                  C.c_void_p(ids.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(_ptr(dw)),
                                  C.c_int64(dw.stride(0) if dense else 0), dtype_code(logits.dtype), _stream()),
            "rf_moe_select")
    return (ids, w, dw) if dense else (ids, w)


def moe_scale_blocks(h: torch.Tensor, dense_w: torch.Tensor, E: int, I: int) -> torch.Tensor:
    """In place: expert block ``e`` (width ``I``) of every row of ``h`` times ``dense_w[:, e]``."""
    N.check(N.lib().rf_moe_scale_blocks(C.c_void_p(h.data_ptr()), C.c_int64(h.stride(0)), C.c_void_p(dense_w.data_ptr()),
                                        C.c_int64(dense_w.stride(0)), h.shape[0], E, I, dtype_code(h.dtype), _stream()),
            "rf_moe_scale_blocks")
    return h


def moe_group(ids: torch.Tensor, w: torch.Tensor, E: int):
    """Bucket the router's picks by expert.  ``ids`` / ``w``: ``[T, k]`` from :func:`moe_select`.  Returns
    ``(slot_of [T*k] int32, token_of_slot [T*k] int32, slot_w [T*k] fp32, tiles int32)``: the sorted row of every
    pick, the token of every sorted row, its routing weight, and the device-side tile list of
    :func:`moe_grouped_gemm` (``tiles[0]`` = number of 128-row blocks)."""
    T, k = ids.shape
    dev = ids.device
    slot_of = torch.empty(T * k, dtype=torch.int32, device=dev)
    token_of_slot = torch.zeros(T * k, dtype=torch.int32, device=dev)
    slot_w = torch.zeros(T * k, dtype=torch.float32, device=dev)
    tiles = torch.zeros(1 + 4 * (T * k // 128 + E + 1), dtype=torch.int32, device=dev)
    N.check(N.lib().rf_moe_group(C.c_void_p(ids.data_ptr()), C.c_void_p(w.data_ptr()), T, k, E, C.c_void_p(slot_of.data_ptr()),
                                 C.c_void_p(token_of_slot.data_ptr()), C.c_void_p(slot_w.data_ptr()),
                                 C.c_void_p(tiles.data_ptr()), _stream()), "rf_moe_group")
    return slot_of, token_of_slot, slot_w, tiles


def moe_grouped_gemm(x: torch.Tensor, bank: torch.Tensor, tiles: torch.Tensor, *, n: int, k: int, bank_rows: int,
                     bank_k: int, expert_rows: int = 0, expert_k: int = 0, dual: bool = False, act: Optional[str] = None,
                     row_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[s] = act(x[s] @ W_e.T) * row_scale[s]`` for every sorted row ``s`` of every expert ``e`` (see
    :func:`moe_group`).  ``bank`` is the ``pack_weight`` image of the whole expert bank: ``bank_rows`` rows per section
    (GLU banks have two sections: gates, then ups) and ``bank_k`` columns.  Experts are ``expert_rows`` rows apart
    (up / gate projection: a multiple of 128) or ``expert_k`` columns apart (down projection: a multiple of 64)."""
    S = x.shape[0]
    assert x.stride(1) == 1 and (expert_rows % 128 == 0) and (expert_k % 64 == 0)
    if out is None:
        out = torch.zeros((S, n), dtype=x.dtype, device=x.device)
    a = N.RfMoeGroupedGemm()
    a.x, a.ldx, a.w, a.out, a.ldo = x.data_ptr(), x.stride(0), bank.data_ptr(), out.data_ptr(), out.stride(0)
    a.row_scale, a.tiles = _ptr(row_scale), tiles.data_ptr()
    a.max_rows, a.N, a.K, a.dual, a.act = S, n, k, int(dual), ACT[act]
    a.bank_section_row_tiles = (bank_rows + 127) // 128
    a.bank_kb_total = (bank_k + 63) // 64
    a.rt_per_expert, a.kb_per_expert = expert_rows // 128, expert_k // 64
    a.dtype, a.status = dtype_code(x.dtype), _ptr(status)
    N.check(N.lib().rf_moe_grouped_gemm(C.byref(a), _stream()), "rf_moe_grouped_gemm")
    return out


def moe_combine(out: torch.Tensor, y: torch.Tensor, slot_of: torch.Tensor, k: int) -> torch.Tensor:
    """In place: ``out[t] += sum_j y[slot_of[t*k + j]]`` (fp32 sum in pick order, one rounding)."""
    T, H = out.shape
    N.check(N.lib().rf_moe_combine(C.c_void_p(out.data_ptr()), C.c_int64(out.stride(0)), C.c_void_p(y.data_ptr()),
                                   C.c_int64(y.stride(0)), C.c_void_p(slot_of.data_ptr()), T, k, H, dtype_code(out.dtype),
                                   _stream()), "rf_moe_combine")
    return out
