"""Python face of the native transformer-stack executor (``csrc/models/stack.{h,cu}``).

``NativeStack`` owns one native handle: per-layer weight pointers (the tensors are kept alive
here), the static activation arena and the status block.  Families differ only by the
``StackSpec`` they pass (norm kind, QK-norm, rope, GLU vs plain MLP, biases, gated residual,
paged vs in-buffer KV), which is how the reference's one-class-per-family fused runtimes
(``src/fused/*.cpp``) collapse into one executor here.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import _native as N
from ..ops import kernels as K
from .errors import RPUBackendError

NORM_KIND = {"rms": 0, "rms_gemma": 1, "layernorm": 2, "adarms": 3}
MLP_KIND = {"swiglu": 0, "geglu_tanh": 1, "gelu_tanh": 2, "gelu_erf": 3, "silu": 4}


@dataclass
class StackSpec:
    layers: int
    hidden: int
    heads: int                 # local query heads
    kv_heads: int              # local kv heads
    head_dim: int              # padded head dim (64 / 128 / 256)
    inter: int                 # local intermediate size
    norm: str = "rms"
    mlp: str = "swiglu"
    eps: float = 1e-6
    qk_norm: bool = False
    rope_before_norm: bool = False
    rot_dim: int = 0           # 0: no rope
    gated_residual: bool = False
    sandwich_norm: bool = False
    paged_kv: bool = False
    causal: bool = False
    window: int = 0
    true_head_dim: int = 0     # unpadded head dim for the softmax scale
    attn_scale: float = 0.0
    max_tokens: int = 1024
    max_seqs: int = 1
    vocab_local: int = 0
    vocab_offset: int = 0
    tp_world: int = 1
    tp_rank: int = 0
    weights_int8: bool = False
    decode_gemv_max_m: int = 0
    packed: bool = True        # linear weights in the tile-major layout of ops.kernels.pack_weight
    attn_gate: bool = False
    # sparse MoE MLP (dense-einsum form): `inter` is then experts * expert_inter + the shared expert's width
    moe_experts: int = 0
    moe_top_k: int = 0
    moe_expert_inter: int = 0
    moe_score_fn: str = "sigmoid"
    moe_norm_topk: bool = True
    moe_routed_scale: float = 1.0


LAYER_FIELDS = ("norm1_w", "norm1_b", "wqkv", "bqkv", "sqkv", "q_norm_w", "k_norm_w", "wo", "bo", "so", "norm2_w",
                "norm2_b", "w_up", "b_up", "s_up", "w_down", "b_down", "s_down", "post_attn_norm_w", "post_mlp_norm_w",
                "moe_router_w", "moe_router_bias")


def pad_heads(w: torch.Tensor, heads: int, hd: int, hd_pad: int, dim: int) -> torch.Tensor:
    """Zero-pad every head of a projection from ``hd`` to ``hd_pad`` along ``dim`` (0: output rows of
    q/k/v or a bias vector, 1: input columns of the output projection).  Zero rows/columns leave
    the attention result unchanged, so odd head sizes (72, 80) run on the 128-wide kernels."""
    if hd == hd_pad:
        return w
    if w.dim() == 1:
        out = w.new_zeros(heads, hd_pad)
        out[:, :hd] = w.view(heads, hd)
        return out.reshape(-1)
    if dim == 0:
        out = w.new_zeros(heads, hd_pad, w.shape[1])
        out[:, :hd] = w.view(heads, hd, w.shape[1])
        return out.reshape(heads * hd_pad, w.shape[1])
    out = w.new_zeros(w.shape[0], heads, hd_pad)
    out[:, :, :hd] = w.view(w.shape[0], heads, hd)
    return out.reshape(w.shape[0], heads * hd_pad)


class NativeStack:
    def __init__(self, spec: StackSpec, layer_weights: Sequence[Dict[str, torch.Tensor]], *, device="cuda",
                 dtype=torch.float16, final_norm_w: Optional[torch.Tensor] = None,
                 final_norm_b: Optional[torch.Tensor] = None, lm_head: Optional[torch.Tensor] = None,
                 lm_head_scale: Optional[torch.Tensor] = None, kv_cache=None, comm=None,
                 twin_layer_weights: Optional[Sequence[Dict[str, torch.Tensor]]] = None,
                 twin_final_norm_w: Optional[torch.Tensor] = None):
        if len(layer_weights) != spec.layers:
            raise RPUBackendError(f"expected {spec.layers} layer weight sets, got {len(layer_weights)}")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        lib = N.lib()
        sc = N.RfStackConfig()
        sc.layers, sc.hidden, sc.Hq, sc.Hkv, sc.hd, sc.inter = (spec.layers, spec.hidden, spec.heads, spec.kv_heads,
                                                                spec.head_dim, spec.inter)
        sc.rot_dim, sc.norm_kind, sc.mlp_kind, sc.eps = spec.rot_dim, NORM_KIND[spec.norm], MLP_KIND[spec.mlp], spec.eps
        sc.qk_norm, sc.rope_before_norm = int(spec.qk_norm), int(spec.rope_before_norm)
        sc.gated_residual, sc.sandwich_norm = int(spec.gated_residual), int(spec.sandwich_norm)
        sc.paged_kv, sc.causal, sc.window = int(spec.paged_kv), int(spec.causal), spec.window
        sc.attn_scale, sc.true_hd = spec.attn_scale, spec.true_head_dim or spec.head_dim
        sc.dtype = K.dtype_code(dtype)
        sc.max_tokens, sc.max_seqs = spec.max_tokens, spec.max_seqs
        sc.vocab_local, sc.vocab_offset = spec.vocab_local, spec.vocab_offset
        sc.tp_world, sc.tp_rank = spec.tp_world, spec.tp_rank
        sc.weights_int8, sc.decode_gemv_max_m = int(spec.weights_int8), spec.decode_gemv_max_m
        sc.weights_packed, sc.attn_gate = int(spec.packed), int(spec.attn_gate)
        sc.moe_experts, sc.moe_top_k, sc.moe_expert_inter = spec.moe_experts, spec.moe_top_k, spec.moe_expert_inter
        sc.moe_score_fn = {"sigmoid": 0, "softmax": 1}[spec.moe_score_fn]
        sc.moe_norm_topk, sc.moe_routed_scale = int(spec.moe_norm_topk), spec.moe_routed_scale
        h = lib.rf_stack_create(C.byref(sc))
        if h < 0:
            N.check(-1, "rf_stack_create")
        self.handle = C.c_int64(h)
        self._keep: List[torch.Tensor] = []
        self.cache = kv_cache
        if twin_layer_weights is not None and len(twin_layer_weights) != spec.layers:
            raise RPUBackendError(f"expected {spec.layers} twin layer weight sets, got {len(twin_layer_weights)}")
        sets = [(l, lw, False) for l, lw in enumerate(layer_weights)]
        sets += [(l, lw, True) for l, lw in enumerate(twin_layer_weights or ())]
        for l, lw, is_twin in sets:
            w = N.RfLayerWeights()
            glu = spec.mlp in ("swiglu", "geglu_tanh")
            for f in LAYER_FIELDS:
                t = lw.get(f)
                if t is not None:
                    d = self._dev(t)
                    if f == "moe_router_bias":          # fp32 whatever the stack's dtype
                        self._keep.pop()
                        d = t.to(self.device, torch.float32).contiguous()
                        self._keep.append(d)
                    if spec.packed and f in ("wqkv", "wo", "w_up", "w_down", "moe_router_w"):
                        self._keep.pop()
                        d = K.pack_weight(d, 2 if (f == "w_up" and glu) else 1)
                        self._keep.append(d)
                    setattr(w, f, d.data_ptr())
            if spec.paged_kv:
                if kv_cache is None:
                    raise RPUBackendError("a paged-KV stack needs a kv_cache")
                w.k_pool, w.v_pool = kv_cache.layer_ptrs(l)
            if is_twin:      # second weight set of the layer: rows at and beyond forward(twin_split=...) run through it
                N.check(lib.rf_stack_set_twin_layer(self.handle, l, C.byref(w)), "rf_stack_set_twin_layer")
            else:
                N.check(lib.rf_stack_set_layer(self.handle, l, C.byref(w)), "rf_stack_set_layer")
        if twin_final_norm_w is not None:
            tf = self._dev(twin_final_norm_w)
            N.check(lib.rf_stack_set_twin_head(self.handle, C.c_void_p(tf.data_ptr())), "rf_stack_set_twin_head")
        if final_norm_w is not None:
            fw = self._dev(final_norm_w)
            fb = self._dev(final_norm_b) if final_norm_b is not None else None
            lm = self._dev(lm_head) if lm_head is not None else None
            if lm is not None and spec.packed:
                self._keep.pop()
                lm = K.pack_weight(lm)
                self._keep.append(lm)
            ls = self._dev(lm_head_scale) if lm_head_scale is not None else None
            N.check(lib.rf_stack_set_head(self.handle, C.c_void_p(fw.data_ptr()),
                                          C.c_void_p(None if fb is None else fb.data_ptr()),
                                          C.c_void_p(None if lm is None else lm.data_ptr()),
                                          C.c_void_p(None if ls is None else ls.data_ptr())), "rf_stack_set_head")
        nbytes = lib.rf_stack_arena_bytes(self.handle)
        self.arena = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=self.device)
        base = (self.arena.data_ptr() + 1023) // 1024 * 1024
        N.check(lib.rf_stack_bind_arena(self.handle, C.c_void_p(base), C.c_uint64(nbytes)), "rf_stack_bind_arena")
        off = lib.rf_stack_status_ptr(self.handle) - self.arena.data_ptr()
        self.status = self.arena[off:off + 32].view(torch.int32)
        if comm is not None:
            cc = comm.stack_comm()
            N.check(lib.rf_stack_set_comm(self.handle, C.byref(cc)), "rf_stack_set_comm")
        self.comm = comm

    def _dev(self, t: torch.Tensor) -> torch.Tensor:
        t = t.to(self.device, self.dtype if t.is_floating_point() else t.dtype).contiguous()
        self._keep.append(t)
        return t

    def bind_cache(self, cache) -> None:
        lib = N.lib()
        for l in range(self.spec.layers):
            k, v = cache.layer_ptrs(l)
            N.check(lib.rf_stack_set_kv(self.handle, l, C.c_void_p(k), C.c_void_p(v)), "rf_stack_set_kv")
        self.cache = cache

    @staticmethod
    def _p(t: Optional[torch.Tensor]):
        return None if t is None else t.data_ptr()

    def forward(self, hidden: torch.Tensor, *, kv_len: torch.Tensor, max_kv_len: int,
                q_start: Optional[torch.Tensor] = None, q_len: Optional[torch.Tensor] = None, max_q_len: int = 1, pos: Optional[torch.Tensor] = None,
                cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                axis_of_freq: Optional[torch.Tensor] = None, decode: bool = False,
                seq_of_tok: Optional[torch.Tensor] = None, cache_pos: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None,
                seg_q: Optional[torch.Tensor] = None, seg_k: Optional[torch.Tensor] = None,
                mod: Optional[torch.Tensor] = None, rows_per_mod: int = 1, layer_range=None,
                deepstack: Optional[Sequence[Optional[torch.Tensor]]] = None,
                deepstack_rows: Optional[torch.Tensor] = None, taps: Optional[Dict[int, torch.Tensor]] = None,
                kv_start: Optional[torch.Tensor] = None, twin_split: int = 0) -> torch.Tensor:
        """Run the layer loop in place on ``hidden`` ``[tokens, hidden]`` (all metadata int32, device)."""
        f = N.RfStackForward()
        T = hidden.shape[0]
        f.hidden, f.tokens, f.decode = hidden.data_ptr(), T, int(decode)
        if pos is not None:
            f.pos, f.pos_stride = pos.data_ptr(), (1 if pos.dim() == 1 else pos.shape[1])
        f.cos, f.sin, f.axis_of_freq = self._p(cos), self._p(sin), self._p(axis_of_freq)
        f.seq_of_tok, f.cache_pos = self._p(seq_of_tok), self._p(cache_pos)
        f.num_seqs = kv_len.numel()
        f.q_start, f.q_len, f.kv_len, f.kv_start = self._p(q_start), self._p(q_len), self._p(kv_len), self._p(kv_start)
        f.max_q_len, f.max_kv_len = max_q_len, max_kv_len
        if page_table is not None:
            f.page_table, f.pt_stride = page_table.data_ptr(), page_table.stride(0)
            f.pool_pages = self.cache.num_pages
        if mask is not None:
            assert mask.dtype in (torch.uint8, torch.bool) and mask.stride(-1) == 1
            f.mask, f.mask_ld = mask.data_ptr(), mask.stride(-2)
            f.mask_seq_stride = mask.stride(0) if mask.dim() == 3 else 0
        f.seg_q, f.seg_k = self._p(seg_q), self._p(seg_k)
        if mod is not None:
            f.mod, f.rows_per_mod = mod.data_ptr(), rows_per_mod
        if layer_range is not None:
            f.layer_begin, f.layer_end = layer_range
        f.twin_split = int(twin_split)
        keep = []
        if deepstack is not None:
            ptrs = torch.tensor([0 if t is None else t.data_ptr() for t in deepstack], dtype=torch.int64)
            keep.append(ptrs)
            f.deepstack = ptrs.data_ptr()          # host array of device pointers
            f.deepstack_rows, f.n_deepstack, f.n_deepstack_rows = deepstack_rows.data_ptr(), len(deepstack), deepstack_rows.numel()
        if taps:
            layers = torch.tensor(sorted(taps), dtype=torch.int32)
            ptrs = torch.tensor([taps[int(l)].data_ptr() for l in layers], dtype=torch.int64)
            keep += [layers, ptrs]
            f.taps, f.tap_layers, f.n_taps = ptrs.data_ptr(), layers.data_ptr(), len(taps)
        N.check(N.lib().rf_stack_forward(self.handle, C.byref(f), C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                "rf_stack_forward")
        return hidden

    def final_norm(self, hidden: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty_like(hidden) if out is None else out
        N.check(N.lib().rf_stack_final_norm(self.handle, C.c_void_p(hidden.data_ptr()), C.c_void_p(out.data_ptr()),
                                            hidden.shape[0], C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                "rf_stack_final_norm")
        return out

    def final_norm_twin(self, hidden: torch.Tensor, twin_split: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Final norm with the stack's own weights on rows ``[0, twin_split)`` and the twin's on the rest."""
        out = torch.empty_like(hidden) if out is None else out
        N.check(N.lib().rf_stack_final_norm_twin(self.handle, C.c_void_p(hidden.data_ptr()), C.c_void_p(out.data_ptr()),
                                                 hidden.shape[0], int(twin_split),
                                                 C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                "rf_stack_final_norm_twin")
        return out

    def check_status(self) -> None:
        torch.cuda.synchronize()
        st = self.status.tolist()
        if st[0] != 0:
            raise RPUBackendError(f"device status {st[:4]} (code, block, kernel, detail)")

    def close(self) -> None:
        if getattr(self, "handle", None) is not None:
            N.lib().rf_stack_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
