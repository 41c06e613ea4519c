"""Causal-LM serving engine on the native transformer-stack runtime.

One engine = one native stack handle (weights packed once, static activation
arena, paged KV pool with 16-token pages) plus the device-resident decode state
(token ids, positions, KV lengths, page table).  A decode step -- embedding,
all layers, final norm, lm_head, arg-max, bookkeeping -- is captured once per
batch size into a CUDA graph and replayed; nothing in it depends on host values.

This is the B200 counterpart of the reference's shared causal-decoder runtime
(``python/rpu_backend/runtime/decoder.py:1012-1519`` install,
``:623-873`` forward) and of its BUILD/REPLAY graph capture
(``python/rpu_backend/graph/_runtime.py:124-340``).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .. import _native as N
from ..models.decoder import DecoderConfig, mrope_axis_of_freq, rope_tables
from ..ops import kernels as K
from ..parallel.tp import CommBuffers, TPContext, kv_head_range, shard_range
from .errors import RPUBackendError

WeightGetter = Callable[[str], torch.Tensor]

NORM_KIND = {"rms": 0, "rms_gemma": 1, "layernorm": 2, "adarms": 3}
MLP_KIND = {"swiglu": 0, "geglu_tanh": 1, "gelu_tanh": 2, "gelu_erf": 3, "silu": 4}


def random_weight_getter(cfg: DecoderConfig, *, seed: int = 0, std: float = 0.02, dtype=torch.float16,
                         device="cuda") -> WeightGetter:
    """Random-init weights generated on demand on ``device`` (one seeded generator per tensor
    name), so an 8B/32B-shape model never exists in host memory and every tensor-parallel
    rank derives identical full tensors before slicing its shard."""
    from ..models.decoder import weight_shapes
    table = {name: (idx, shape, kind) for idx, (name, shape, kind) in enumerate(weight_shapes(cfg))}
    dev = torch.device(device)

    def get(name: str) -> torch.Tensor:
        if name == "lm_head.weight" and name not in table:
            return get("model.embed_tokens.weight")
        idx, shape, kind = table[name]
        if kind == "norm":
            return torch.full(shape, 0.0 if cfg.norm == "rms_gemma" else 1.0, dtype=dtype, device=dev)
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 1_000_003 + idx)
        t = torch.empty(shape, dtype=torch.float32, device=dev) if len(shape) == 1 else None
        if t is not None:
            return (t.normal_(0.0, std, generator=g)).to(dtype)
        out = torch.empty(shape, dtype=dtype, device=dev)
        rows = max(1, (64 << 20) // (shape[1] * 4))
        for r in range(0, shape[0], rows):
            blk = torch.empty((min(rows, shape[0] - r), shape[1]), dtype=torch.float32, device=dev)
            out[r:r + blk.shape[0]] = blk.normal_(0.0, std, generator=g).to(dtype)
        return out

    return get


def quantize_per_channel(w: torch.Tensor, dtype=torch.float16):
    """Symmetric per-output-channel int8 (reference semantics: ``quant/_common.py:10-41``)."""
    amax = w.float().abs().amax(dim=1).clamp(min=1e-8)
    scale = (amax / 127.0).to(dtype)
    scale = torch.where(scale > 0, scale, torch.ones_like(scale))     # all-zero rows (padding): q = 0, scale = 1
    q = torch.round(w.float() / scale.float()[:, None]).clamp(-127, 127).to(torch.int8)
    return q, scale


class DecoderEngine:
    def __init__(self, cfg: DecoderConfig, get_weight: WeightGetter, *, device="cuda", dtype=torch.float16,
                 max_batch: int = 1, max_seq_len: int = 2048, max_prefill_tokens: int = 8192,
                 tp: Optional[TPContext] = None, quant: Optional[str] = None, decode_gemv_max_m: int = 0,
                 hist_steps: int = 4096, kv_cache=None, kv_pool_tokens: Optional[int] = None, w4_group: int = 64):
        if not torch.cuda.is_available():
            raise RPUBackendError("DecoderEngine needs a CUDA device")
        self.cfg, self.dtype = cfg, dtype
        self.tp = tp or TPContext.single(device)
        self.device = torch.device(self.tp.device if self.tp.device is not None else device)
        W, R = self.tp.world, self.tp.rank
        self.max_batch = max_batch
        self.max_tokens = max(max_prefill_tokens, max_batch)
        self.quant = quant
        if quant not in (None, "w8a16", "w4a16"):
            raise RPUBackendError(f"unknown quantisation {quant!r}")
        if w4_group not in (0, 32, 64, 128):
            raise RPUBackendError(f"w4_group must be 0 (per channel), 32, 64 or 128, got {w4_group}")
        self.w4_group = w4_group
        H, hd = cfg.hidden_size, cfg.head_dim
        if cfg.num_heads % W or cfg.intermediate_size % W or cfg.vocab_size % W:
            raise RPUBackendError(f"{cfg.name}: heads/intermediate/vocab do not split over {W} ranks")
        self.Hq = cfg.num_heads // W
        kv0, kv1 = kv_head_range(cfg.num_kv_heads, W, R)
        self.Hkv = kv1 - kv0
        self.inter = cfg.intermediate_size // W
        self.vocab_local = cfg.vocab_size // W
        lib = N.lib()

        sc = N.RfStackConfig()
        sc.layers, sc.hidden, sc.Hq, sc.Hkv, sc.hd, sc.inter = cfg.num_layers, H, self.Hq, self.Hkv, hd, self.inter
        sc.rot_dim, sc.norm_kind, sc.mlp_kind, sc.eps = cfg.rot_dim, NORM_KIND[cfg.norm], MLP_KIND[cfg.mlp], cfg.rms_eps
        sc.qk_norm, sc.paged_kv, sc.causal, sc.true_hd = int(cfg.qk_norm), 1, 1, hd
        sc.dtype = K.dtype_code(dtype)
        sc.max_tokens, sc.max_seqs = self.max_tokens, max_batch
        sc.vocab_local, sc.vocab_offset = self.vocab_local, R * self.vocab_local
        sc.tp_world, sc.tp_rank = W, R
        sc.weights_int8 = 1 if quant in ("w8a16", "w4a16") else 0
        if quant == "w4a16":
            sc.weights_bits, sc.weights_group = 4, w4_group
        sc.decode_gemv_max_m = decode_gemv_max_m
        sc.attn_gate = int(cfg.attn_gate)
        # linear weights live in the tile-major layout (contiguous 16 KB blocks): see ops.kernels.pack_weight
        self.packed = os.environ.get("RF_PACKED_WEIGHTS", "1") != "0" and decode_gemv_max_m == 0
        sc.weights_packed = int(self.packed)
        # Pre-norm weights multiplied into the columns of the projections that follow them (q/k/v, gate/up): the
        # RMSNorm between a residual GEMM and the next projection then needs no kernel of its own at decode sizes
        # (the residual GEMM emits sums of squares, the projection scales its rows).  One GPU, dense decoders, 16-bit
        # weights (quantised engines keep the checkpoint's exact integer weights).
        self.fold_norm = (W == 1 and cfg.norm in ("rms", "rms_gemma") and not any(cfg.is_linear(l) for l in range(cfg.num_layers))
                          and quant is None and getattr(get_weight, "scale", None) is None and self.packed
                          and os.environ.get("RF_FOLD_NORM", "1") != "0")
        sc.norm_folded = int(self.fold_norm)
        sc.gemm_streaming_only = 1          # one GEMM kernel family at every tensor-parallel degree
        # hybrid decoders: which layers own KV pages, and the local Gated-DeltaNet geometry
        self.attn_layers = [l for l in range(cfg.num_layers) if not cfg.is_linear(l)]
        self.kv_index = {l: i for i, l in enumerate(self.attn_layers)}
        self.gdn_layers = [l for l in range(cfg.num_layers) if cfg.is_linear(l)]
        if self.gdn_layers:
            if cfg.gdn_heads_k % W or cfg.gdn_heads_v % W:
                raise RPUBackendError(f"{cfg.name}: linear-attention heads do not split over {W} ranks")
            self.gdn_Hk, self.gdn_Hv = cfg.gdn_heads_k // W, cfg.gdn_heads_v // W
            sc.gdn_Hk, sc.gdn_Hv, sc.gdn_Dk, sc.gdn_Dv, sc.gdn_conv_k = (self.gdn_Hk, self.gdn_Hv, cfg.gdn_dk,
                                                                        cfg.gdn_dv, cfg.gdn_conv)
        h = lib.rf_stack_create(C.byref(sc))
        if h < 0:
            N.check(-1, "rf_stack_create")
        self.handle = C.c_int64(h)

        # ---- KV cache: a PagedKV (or RPUCache) object; replaceable through bind_cache()
        from .kv_cache import PagedKV
        self.cache = kv_cache if kv_cache is not None else PagedKV(len(self.attn_layers), max_batch, max_seq_len,
                                                                     self.Hkv, hd, device=self.device, dtype=dtype,
                                                                     pool_tokens=kv_pool_tokens)
        self._check_cache(self.cache)
        # recurrent + conv state of the linear-attention layers, one slot per sequence of the batch
        self.gdn_conv_state: Dict[int, torch.Tensor] = {}
        self.gdn_rec_state: Dict[int, torch.Tensor] = {}
        for l in self.gdn_layers:
            conv_dim = 2 * self.gdn_Hk * cfg.gdn_dk + self.gdn_Hv * cfg.gdn_dv
            self.gdn_conv_state[l] = torch.zeros((max_batch, cfg.gdn_conv - 1, conv_dim), dtype=dtype, device=self.device)
            self.gdn_rec_state[l] = torch.zeros((max_batch, self.gdn_Hv, cfg.gdn_dk, cfg.gdn_dv), dtype=torch.float32,
                                                device=self.device)

        # ---- weights: packed once, kept alive here
        self._keep: List[torch.Tensor] = []
        self._pack_weights(get_weight, kv0, kv1)

        # ---- arena + comm
        nbytes = lib.rf_stack_arena_bytes(self.handle)
        self.arena = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=self.device)
        base = (self.arena.data_ptr() + 1023) // 1024 * 1024
        N.check(lib.rf_stack_bind_arena(self.handle, C.c_void_p(base), C.c_uint64(nbytes)), "rf_stack_bind_arena")
        off = lib.rf_stack_status_ptr(self.handle) - self.arena.data_ptr()
        self.status = self.arena[off:off + 32].view(torch.int32)
        self.comm: Optional[CommBuffers] = None
        if self.tp.enabled:
            from .control import tp_comm_mode
            if tp_comm_mode() == "nccl":
                raise RPUBackendError("RPU_TP_COMM=nccl: the engine's step has no NCCL path (its all-reduce is the GEMM "
                                      "epilogue); the NCCL implementation of the same models is baseline/eager_tp.py")
            # receive slots of the publish / consume all-reduce (<= 256 rows, fp32 partials at most) and four symmetric
            # [max_tokens, hidden] activation buffers for the prefill-sized row all-reduce; RF_TP_AR=inkernel (the
            # all-reduce inside the GEMM epilogue, A/B timing) needs room for 16-bit partials + results of all rows
            need = W * min(self.max_tokens, 256) * H * 4
            if os.environ.get("RF_TP_AR") == "inkernel":
                need = max(need, (W + 1) * self.max_tokens * H * 2)
            self.comm = CommBuffers(self.tp, need, sym_rows=self.max_tokens, sym_cols=H, sym_elem_bytes=2)
            cc = self.comm.stack_comm()
            N.check(lib.rf_stack_set_comm(self.handle, C.byref(cc)), "rf_stack_set_comm")

        # ---- rope tables and decode state
        cos, sin = rope_tables(cfg, max_seq_len + 16, self.device)
        self.cos, self.sin = cos, sin
        ax = mrope_axis_of_freq(cfg)
        self.axis = ax.to(self.device) if ax is not None else None
        self.pos_stride = 3 if ax is not None else 1
        i32 = dict(dtype=torch.int32, device=self.device)
        # the residual stream: under tensor parallelism it lives in the peer-mapped region, where the owner rank of a
        # row stores the all-reduced row into every rank's copy
        self.hidden = (self.comm.sym_tensor("hidden", dtype) if self.comm is not None
                       else torch.zeros((self.max_tokens, H), dtype=dtype, device=self.device))
        self.ids = torch.zeros(max_batch, **i32)
        self.out_ids = torch.zeros(max_batch, **i32)
        self.out_vals = torch.zeros(max_batch, dtype=torch.float32, device=self.device)
        self.pos = torch.zeros((max_batch, self.pos_stride), **i32)
        self.kv_len = torch.zeros(max_batch, **i32)
        self.step = torch.zeros(1, **i32)
        self.hist_steps = hist_steps
        self.hist = torch.zeros((hist_steps, max_batch), **i32)
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.batch = 0
        self.launches_per_step = 0
        self._hb = 0                         # host heartbeat counter (tensor parallel only)
        self._host_steps = 0
        self.heartbeat_every = int(os.environ.get("RPU_TP_HEARTBEAT_STEPS", "64"))
        if self.tp.enabled:
            self._check_plan_agreement()

    # ------------------------------------------------------------------ weights
    def _dev(self, t: torch.Tensor) -> torch.Tensor:
        t = t.to(self.device, self.dtype if t.is_floating_point() else t.dtype).contiguous()
        self._keep.append(t)
        return t

    def _pack(self, w: torch.Tensor, sections: int) -> torch.Tensor:
        if not self.packed:
            return w
        if self._keep and self._keep[-1] is w:
            self._keep.pop()                 # only the packed image stays resident
        p = K.pack_weight(w, sections)
        self._keep.append(p)
        return p

    def _lin_w4(self, get: WeightGetter, parts, cols, sections: int):
        """One int4 linear: packed checkpoint tensors (``uint8 [out, in/2]`` + group or channel scales) are unpacked, sliced
        and re-packed into the tile-major image; 16-bit tensors are quantised here with this engine's group size."""
        from ..quant.int4_pack import unpack_int4
        scale_of = getattr(get, "scale", None)
        G = self.w4_group
        qs, ss = [], []
        for name, rows in parts:
            if name is None:
                raise RPUBackendError("int4 weights do not take alignment padding rows")
            w = get(name)
            if w.dtype == torch.uint8:
                sc = scale_of(name) if scale_of is not None else None
                if sc is None:
                    raise RPUBackendError(f"packed int4 weight {name!r} has no weight_scale")
                q = unpack_int4(w)
                Kd = q.shape[1]
                sc = sc.reshape(q.shape[0], -1).float()
                g_ck = Kd // sc.shape[1] if sc.shape[1] > 1 else 0
                if g_ck != G:
                    raise RPUBackendError(f"{name!r} was quantised with scale group {g_ck or 'per-channel'}, the engine was "
                                          f"built for {G or 'per-channel'}")
            else:
                wf = w.to(self.device).float()
                Kd = wf.shape[1]
                grp = wf.view(wf.shape[0], Kd // G, G) if G else wf.view(wf.shape[0], 1, Kd)
                sc = (grp.abs().amax(-1) / 7.0).clamp_min(1e-8)
                q = torch.round(grp / sc[..., None]).clamp_(-8, 7).to(torch.int8).view(wf.shape[0], Kd)
            q, sc = q[rows], sc[rows]
            if cols is not None:
                q = q[:, cols]
                if G:
                    c0, c1, _ = cols.indices(Kd)
                    if c0 % G or c1 % G:
                        raise RPUBackendError(f"{name!r}: the tensor-parallel shard [{c0}, {c1}) cuts a scale group of {G}")
                    sc = sc[:, c0 // G:c1 // G]
            qs.append(q.to(self.device))
            ss.append(sc.to(self.device))
        q = qs[0] if len(qs) == 1 else torch.cat(qs, 0)
        sc = ss[0] if len(ss) == 1 else torch.cat(ss, 0)
        if G:
            img = K.pack_weight_int4(q, sc, G, sections=sections, dtype=self.dtype)
            self._keep.append(img)
            return img, img                       # the second pointer only marks the weight as quantised
        img = K.pack_weight_int4(q, sections=sections)
        self._keep.append(img)
        return img, self._dev(sc.reshape(-1).to(self.dtype))

    def _lin(self, get: WeightGetter, parts, cols=None, sections: int = 1, w4: bool = True, col_scale=None):
        """One packed linear: ``parts`` is a list of (tensor name, row slice); the pieces are
        concatenated along the output dim, ``cols`` slices the input dim (row-parallel shards).
        Returns (device weight, device per-channel scale or None).  int8 checkpoints keep their
        stored scales; 16-bit weights are quantised here when the engine runs W8A16."""
        if col_scale is not None:
            # fold a per-input-column factor (a pre-norm's weights) into the matrix before it is packed or quantised
            inner, cs = get, col_scale.to(self.device, torch.float32)

            def get(name, _g=inner):
                t = _g(name)
                if not t.is_floating_point():
                    raise RPUBackendError(f"{name!r} is already quantised: the norm weights cannot be folded into it")
                return (t.to(self.device).float() * cs).to(t.dtype)
        if self.quant == "w4a16" and w4:
            return self._lin_w4(get, parts, cols, sections)
        scale_of = getattr(get, "scale", None)
        ws, ss = [], []
        for name, rows in parts:
            if name is None:                     # ``rows`` all-zero output rows (alignment padding)
                ref = ws[0]
                ws.append(torch.zeros((rows, ref.shape[1]), dtype=ref.dtype, device=ref.device))
                ss.append(None if ss[0] is None else torch.ones(rows, dtype=ss[0].dtype, device=ss[0].device))
                continue
            w = get(name)
            sc = scale_of(name) if (scale_of is not None and w.dtype == torch.int8) else None
            w = w[rows]
            if cols is not None:
                w = w[:, cols]
            ws.append(w)
            ss.append(None if sc is None else sc[rows])
        w = ws[0] if len(ws) == 1 else torch.cat(ws, 0)
        if w.dtype == torch.int8:
            if any(x is None for x in ss):
                raise RPUBackendError(f"int8 weight {parts[0][0]!r} has no weight_scale")
            if self.quant not in ("w8a16", "w4a16"):
                raise RPUBackendError("int8 weights need quant='w8a16'")
            sc = ss[0] if len(ss) == 1 else torch.cat(ss, 0)
            sc_d = self._dev(sc.to(self.dtype))
            return self._pack(self._dev(w), sections), sc_d
        if self.quant == "w8a16":
            q, sc = quantize_per_channel(w.to(self.device), self.dtype)
            sc_d = self._dev(sc)
            return self._pack(self._dev(q), sections), sc_d
        return self._pack(self._dev(w), sections), None

    def _pack_weights(self, get: WeightGetter, kv0: int, kv1: int) -> None:
        cfg, lib = self.cfg, N.lib()
        W, R = self.tp.world, self.tp.rank
        hd = cfg.head_dim
        q0, q1 = shard_range(cfg.num_heads, W, R)
        i0, i1 = shard_range(cfg.intermediate_size, W, R)
        v0, v1 = shard_range(cfg.vocab_size, W, R)
        ptr = lambda t: None if t is None else t.data_ptr()
        qs, ks, isl = slice(q0 * hd, q1 * hd), slice(kv0 * hd, kv1 * hd), slice(i0, i1)
        full = slice(None)
        for l in range(cfg.num_layers):
            p = f"model.layers.{l}."
            bqkv = None
            if cfg.attention_bias:
                bq, bk, bv = (get(p + f"self_attn.{n}_proj.bias") for n in "qkv")
                bqkv = self._dev(torch.cat((bq[qs], bk[ks], bv[ks]), 0))
            lw = N.RfLayerWeights()

            def norm_cols(name, _p=p):
                if not self.fold_norm:
                    return None
                w = get(_p + name).float()
                return 1.0 + w if cfg.norm == "rms_gemma" else w
            if cfg.is_linear(l):
                t_qkv, s_qkv, t_o, s_o = self._pack_gdn(get, l, lw)
            else:
                if cfg.attn_gate:
                    # q_proj rows are [head][query hd | gate hd]: queries first, gates behind K and V
                    idx = torch.arange(cfg.num_heads * 2 * hd).view(cfg.num_heads, 2, hd)[q0:q1]
                    q_rows, g_rows = idx[:, 0].reshape(-1), idx[:, 1].reshape(-1)
                    parts = [(p + "self_attn.q_proj.weight", q_rows), (p + "self_attn.k_proj.weight", ks),
                             (p + "self_attn.v_proj.weight", ks), (p + "self_attn.q_proj.weight", g_rows)]
                else:
                    parts = [(p + "self_attn.q_proj.weight", qs), (p + "self_attn.k_proj.weight", ks),
                             (p + "self_attn.v_proj.weight", ks)]
                t_qkv, s_qkv = self._lin(get, parts, col_scale=norm_cols("input_layernorm.weight"))
                t_o, s_o = self._lin(get, [(p + "self_attn.o_proj.weight", full)], cols=qs)
            t_gu, s_gu = self._lin(get, [(p + "mlp.gate_proj.weight", isl), (p + "mlp.up_proj.weight", isl)], sections=2,
                                   col_scale=norm_cols("post_attention_layernorm.weight"))
            t_d, s_d = self._lin(get, [(p + "mlp.down_proj.weight", full)], cols=isl)
            lw.wqkv, lw.sqkv, lw.bqkv = ptr(t_qkv), ptr(s_qkv), ptr(bqkv)
            lw.wo, lw.so = ptr(t_o), ptr(s_o)
            lw.w_up, lw.s_up = ptr(t_gu), ptr(s_gu)
            lw.w_down, lw.s_down = ptr(t_d), ptr(s_d)
            lw.norm1_w = ptr(self._dev(get(p + "input_layernorm.weight")))
            lw.norm2_w = ptr(self._dev(get(p + "post_attention_layernorm.weight")))
            if cfg.qk_norm and not cfg.is_linear(l):
                lw.q_norm_w = ptr(self._dev(get(p + "self_attn.q_norm.weight")))
                lw.k_norm_w = ptr(self._dev(get(p + "self_attn.k_norm.weight")))
            if not cfg.is_linear(l):
                lw.k_pool, lw.v_pool = self.cache.layer_ptrs(self.kv_index[l])
            N.check(lib.rf_stack_set_layer(self.handle, l, C.byref(lw)), "rf_stack_set_layer")
        emb = get("model.embed_tokens.weight")
        self.embed_scale_rows = None
        if emb.dtype == torch.int8:
            sc = getattr(get, "scale")("model.embed_tokens.weight")
            self.embed = self._dev(emb)
            self.embed_scale_rows = self._dev(sc.to(self.dtype))
        else:
            self.embed = self._dev(emb)
        names = getattr(get, "names", None)
        has_head = (names is None and not cfg.tie_embeddings) or (names is not None and "lm_head.weight" in names)
        head_name = "lm_head.weight" if has_head else "model.embed_tokens.weight"
        t_lm, s_lm = self._lin(get, [(head_name, slice(v0, v1))], w4=False)     # the head stays 16-bit under W4A16
        self.final_norm = self._dev(get("model.norm.weight"))
        N.check(lib.rf_stack_set_head(self.handle, C.c_void_p(self.final_norm.data_ptr()), None,
                                      C.c_void_p(t_lm.data_ptr()), C.c_void_p(ptr(s_lm))), "rf_stack_set_head")
        del emb
        torch.cuda.empty_cache()

    def _pack_gdn(self, get: WeightGetter, l: int, lw) -> tuple:
        """Gated-DeltaNet layer: fused input projection ``[q | k | v | z | b | a]`` (b and a padded to 8
        rows), depthwise conv taps, decay parameters, gated-norm weight, state pointers."""
        cfg = self.cfg
        W, R = self.tp.world, self.tp.rank
        p = f"model.layers.{l}.linear_attn."
        Dk, Dv = cfg.gdn_dk, cfg.gdn_dv
        k0, k1 = shard_range(cfg.gdn_heads_k, W, R)
        v0, v1 = shard_range(cfg.gdn_heads_v, W, R)
        key_dim = cfg.gdn_heads_k * Dk
        q_rows = slice(k0 * Dk, k1 * Dk)
        k_rows = slice(key_dim + k0 * Dk, key_dim + k1 * Dk)
        v_rows = slice(2 * key_dim + v0 * Dv, 2 * key_dim + v1 * Dv)
        z_rows, h_rows = slice(v0 * Dv, v1 * Dv), slice(v0, v1)
        pad = (self.gdn_Hv + 7) // 8 * 8 - self.gdn_Hv
        qkv = p + "in_proj_qkv.weight"
        parts = [(qkv, q_rows), (qkv, k_rows), (qkv, v_rows), (p + "in_proj_z.weight", z_rows), (p + "in_proj_b.weight", h_rows)]
        parts += [(None, pad)] if pad else []
        parts += [(p + "in_proj_a.weight", h_rows)] + ([(None, pad)] if pad else [])
        t_in, s_in = self._lin(get, parts)
        t_o, s_o = self._lin(get, [(p + "out_proj.weight", slice(None))], cols=z_rows)
        conv = get(p + "conv1d.weight")
        conv = conv.reshape(conv.shape[0], -1)
        conv = torch.cat((conv[q_rows], conv[k_rows], conv[v_rows]), 0)
        f32 = lambda t: t.to(self.device, torch.float32).contiguous()
        a_log, dtb = f32(get(p + "A_log")[h_rows]), f32(get(p + "dt_bias")[h_rows])
        self._keep += [a_log, dtb]
        lw.mixer = 1
        lw.gdn_conv_w = self._dev(conv).data_ptr()
        lw.gdn_A_log, lw.gdn_dt_bias = a_log.data_ptr(), dtb.data_ptr()
        lw.gdn_norm_w = self._dev(get(p + "norm.weight")).data_ptr()
        lw.gdn_conv_state = self.gdn_conv_state[l].data_ptr()
        lw.gdn_rec_state = self.gdn_rec_state[l].data_ptr()
        return t_in, s_in, t_o, s_o

    def advance_lengths(self, n_steps: int) -> None:
        """Account for ``n_steps`` graph replays issued outside :meth:`decode`."""
        self.cache.lengths[:self.batch] += n_steps

    def reserve_steps(self, n_steps: int) -> None:
        """Give every sequence of the batch KV pages for ``n_steps`` more decode steps (a caller that replays
        the captured graph itself calls this first; :meth:`decode` does it on its own)."""
        self.cache.ensure_batch(self.batch, n_steps + 1)

    def _liveness(self) -> None:
        """Tensor-parallel ranks confirm on the host, between steps and with no kernel of this call in flight yet,
        that every peer is still there: a dead peer is then an exception here, not a one-second in-kernel flag
        timeout per waiting kernel."""
        if self.tp.enabled:
            self._hb += 1
            self.tp.heartbeat(self._hb)
            self.tp.check_peers(self._hb)

    def _check_plan_agreement(self) -> None:
        """Every rank must launch the same grids on the shared flag arrays: compare a digest of what decides the launch
        plans (model geometry, dtype, quantisation, batch / token envelope, weight layout, planner environment) across
        ranks once, at construction.  A mismatch (say an environment override on one rank) would otherwise only show
        up as a peer-wait timeout inside a kernel."""
        import hashlib
        c = self.cfg
        # every kernel-selection switch of this library starts with RF_ (RF_TP_REPORT only names a test's report file)
        env = {k: v for k, v in os.environ.items() if k.startswith("RF_") and k != "RF_TP_REPORT"}
        desc = repr((c.name, c.num_layers, c.hidden_size, c.num_heads, c.num_kv_heads, c.head_dim, c.intermediate_size,
                     c.vocab_size, str(self.dtype), self.quant, self.max_batch, self.max_tokens, self.packed,
                     self.tp.world, sorted(env.items())))
        digest = hashlib.sha256(desc.encode()).hexdigest()[:16]
        seen = self.tp.all_gather_object(digest)
        if len(set(seen)) != 1:
            raise RPUBackendError(f"tensor-parallel ranks disagree on the launch plan inputs (digests by rank: {seen}); "
                                  "check per-rank environment overrides and constructor arguments")

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._keep)

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def check_status(self) -> None:
        """Raise if any kernel recorded a timeout / bad-argument code (reads 8 ints from the device)."""
        torch.cuda.synchronize()
        st = self.status.tolist()
        if st[0] != 0:
            raise RPUBackendError(f"device status {st[:4]} (code, block, kernel, detail)")
        if self.comm is not None and int(self.comm.status[0]) != 0:
            raise RPUBackendError(f"peer wait timed out: {self.comm.status.tolist()[:4]}")

    def _check_cache(self, cache) -> None:
        want = (len(self.attn_layers), self.Hkv, self.cfg.head_dim)
        got = (cache.num_layers, cache.num_kv_heads, cache.head_dim)
        if want != got or cache.dtype != self.dtype or cache.batch_size > self.max_batch:
            raise RPUBackendError(f"KV cache geometry {got}/{cache.dtype}/batch {cache.batch_size} does not match the "
                                  f"model {want}/{self.dtype}/max_batch {self.max_batch}")

    def bind_cache(self, cache) -> None:
        """Make ``cache`` the engine's KV store (pool pointers are re-bound; captured graphs that
        baked the previous pool are dropped)."""
        if cache is self.cache:
            return
        self._check_cache(cache)
        lib = N.lib()
        for l in self.attn_layers:
            k, v = cache.layer_ptrs(self.kv_index[l])
            N.check(lib.rf_stack_set_kv(self.handle, l, C.c_void_p(k), C.c_void_p(v)), "rf_stack_set_kv")
        states = getattr(cache, "linear_states", None)
        if self.gdn_layers and states is not None:
            for i, l in enumerate(self.gdn_layers):
                conv, rec = states(i)
                N.check(lib.rf_stack_set_state(self.handle, l, C.c_void_p(conv.data_ptr()), C.c_void_p(rec.data_ptr())),
                        "rf_stack_set_state")
                self.gdn_conv_state[l], self.gdn_rec_state[l] = conv, rec
        self.cache = cache
        self.graphs.clear()

    @property
    def max_seq_len(self) -> int:
        return self.cache.max_seq_len

    @max_seq_len.setter
    def max_seq_len(self, v) -> None:
        self._max_seq_len_hint = v

    def reset(self) -> None:
        for s in range(self.cache.batch_size):
            self.cache.release(s)
        self.step.zero_()
        self.batch = 0

    def _embed(self, ids: torch.Tensor, n: int) -> None:
        K.embedding(self.embed, ids, out=self.hidden[:n], scale=self.cfg.embed_scale, row_scale=self.embed_scale_rows)

    def _head(self, rows: int, row_idx: Optional[torch.Tensor], logits_out: Optional[torch.Tensor] = None) -> None:
        N.check(N.lib().rf_stack_head(self.handle, C.c_void_p(self.hidden.data_ptr()),
                                      C.c_void_p(None if row_idx is None else row_idx.data_ptr()), rows,
                                      C.c_void_p(self.out_ids.data_ptr()), C.c_void_p(self.out_vals.data_ptr()),
                                      C.c_void_p(None if logits_out is None else logits_out.data_ptr()),
                                      self._stream()), "rf_stack_head")
        if self.comm is not None:
            self.comm.argmax_merge(self.out_vals, self.out_ids, rows)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, prompts: Sequence[torch.Tensor], **kw):
        """Start sequences 0..B-1 from empty with ``prompts``; see :meth:`extend`."""
        self.reset()
        return self.extend(prompts, **kw)

    @torch.no_grad()
    def extend(self, tokens: Sequence[torch.Tensor], *, return_logits: bool = False, logits_rows: int = 1,
               inputs_embeds: Optional[Sequence[torch.Tensor]] = None,
               positions3: Optional[Sequence[torch.Tensor]] = None,
               deepstack: Optional[Sequence[Optional[tuple]]] = None):
        """Append ``tokens[s]`` (1-D int tensors, host or device) to sequence ``s`` at its current
        length and return the greedy next token of every sequence ([B] int32 on the device; with
        ``return_logits`` also the last-row logits of this rank's vocab shard).  Long inputs run as
        several packed varlen launches of at most ``max_prefill_tokens`` rows (chunked prefill);
        the engine is left ready for :meth:`decode`.

        ``inputs_embeds[s]`` ``[L, hidden]`` replaces the embedding lookup (vision rows already spliced
        in); ``positions3[s]`` ``[3, L]`` are M-RoPE positions; ``deepstack[s] = (rows, feats)`` adds
        ``feats[l][i]`` to the hidden row ``rows[i]`` of sequence ``s`` after layer ``l`` (DeepStack).

        ``logits_rows`` (with ``return_logits``): 1 returns ``[B, vocab]`` of the last rows; ``k > 1`` or ``0`` (all) returns a
        list with one ``[rows_s, vocab]`` tensor per sequence holding its last ``k`` (or all) new rows."""
        B = len(tokens)
        cache = self.cache
        if B > cache.batch_size:
            raise RPUBackendError(f"batch {B} exceeds the cache's batch_size {cache.batch_size}")
        self._liveness()
        starts = [int(cache.lengths[s]) for s in range(B)]
        lens = [int(p.numel()) for p in tokens]
        for s, L in enumerate(lens):
            if L < 1:
                raise RPUBackendError("every sequence needs at least one new token")
            cache.check_fits(s, L + 1)
        for s, L in enumerate(lens):              # pages for the new tokens and the first decode step
            cache.ensure(s, starts[s] + L + 1)
        cache.sync_table()
        logits_all = torch.empty((B, self.vocab_local), dtype=self.dtype, device=self.device) if return_logits else None
        first = torch.zeros(B, dtype=torch.int32, device=self.device)
        chunk: List[tuple] = []
        used = 0
        items: List[List[tuple]] = []
        for s, L in enumerate(lens):
            off = 0
            while off < L:
                take = min(L - off, self.max_tokens - used)
                if take == 0:
                    items.append(chunk)
                    chunk, used = [], 0
                    continue
                chunk.append((s, off, take))
                used += take
                off += take
        if chunk:
            items.append(chunk)
        row_logits = None
        if return_logits and logits_rows != 1:
            row_logits = {"keep": int(logits_rows), "out": [[] for _ in range(B)]}
        for ch in items:
            self._prefill_chunk(ch, tokens, lens, starts, first, logits_all, inputs_embeds, positions3, deepstack, row_logits)
        self.batch = B
        for s, L in enumerate(lens):
            cache.lengths[s] = starts[s] + L
        # decode state: the token to feed next is `first`, at position = new length
        self.ids[:B].copy_(first)
        new_len = torch.from_numpy(cache.lengths[:B].astype("int32"))
        if self.device.type == "cuda":
            new_len = new_len.pin_memory()
        new_len = new_len.to(self.device, non_blocking=True)
        if positions3 is not None:
            # generation continues one past the largest position on all three axes
            nxt = torch.stack([p.max().to(self.device) + 1 for p in positions3]).to(torch.int32)
            self.pos[:B].copy_(nxt[:, None].expand(B, self.pos_stride))
        else:
            self.pos[:B].copy_(new_len[:, None].expand(B, self.pos_stride))
        self.kv_len[:B].copy_(new_len + 1)
        if row_logits is not None:
            return first, [torch.cat(parts) if parts else logits_all.new_empty((0, self.vocab_local)) for parts in row_logits["out"]]
        return (first, logits_all) if return_logits else first

    def _prefill_chunk(self, ch, prompts, lens, starts, first, logits_all, inputs_embeds, positions3,
                       deepstack=None, row_logits=None) -> None:
        T = sum(c[2] for c in ch)
        n = len(ch)
        meta = torch.empty((6, max(n, 1)), dtype=torch.int32)
        tokmeta = torch.empty((2, T), dtype=torch.int32)
        ids_host = torch.empty(T, dtype=torch.int32)
        o = 0
        emb_rows = []
        pos3 = []
        ds_rows, ds_feats = [], None
        for j, (s, off, cnt) in enumerate(ch):
            base = starts[s]
            meta[0, j], meta[1, j], meta[2, j] = o, cnt, base + off + cnt   # q_start, q_len, kv_len
            meta[3, j] = s
            meta[4, j] = o + cnt - 1
            meta[5, j] = 1 if (base + off) == 0 else 0        # starts from an empty recurrent state
            tokmeta[0, o:o + cnt] = s
            tokmeta[1, o:o + cnt] = torch.arange(base + off, base + off + cnt, dtype=torch.int32)
            ids_host[o:o + cnt] = prompts[s][off:off + cnt].to("cpu", torch.int32)
            if inputs_embeds is not None:
                emb_rows.append(inputs_embeds[s][off:off + cnt])
            if positions3 is not None:
                pos3.append(positions3[s][:, off:off + cnt].t())
            if deepstack is not None and deepstack[s] is not None:
                rows_s, feats_s = deepstack[s]
                rows_s = rows_s.to("cpu", torch.int64)
                sel = ((rows_s >= off) & (rows_s < off + cnt)).nonzero().flatten()
                if sel.numel():
                    ds_rows.append(rows_s[sel] - off + o)
                    if ds_feats is None:
                        ds_feats = [[] for _ in feats_s]
                    for l, ft in enumerate(feats_s):
                        ds_feats[l].append(ft.to(self.device, self.dtype)[sel.to(self.device)])
            o += cnt
        meta_d = meta.pin_memory().to(self.device, non_blocking=True)
        tok_d = tokmeta.pin_memory().to(self.device, non_blocking=True)
        ids_d = ids_host.pin_memory().to(self.device, non_blocking=True)
        # the page table the kernels see is indexed by chunk-local sequence number
        pt = self.cache.page_table[meta_d[3].long()].contiguous()
        seq_local = torch.repeat_interleave(torch.arange(n, dtype=torch.int32, device=self.device), meta_d[1].long())
        if inputs_embeds is not None:
            self.hidden[:T].copy_(torch.cat(emb_rows).to(self.device, self.dtype))
        else:
            self._embed(ids_d, T)
        if positions3 is not None:
            pos_d = torch.cat(pos3).to(self.device, torch.int32).contiguous()
            cache_pos = tok_d[1].contiguous()
        else:
            pos_d = tok_d[1].contiguous() if self.pos_stride == 1 else tok_d[1][:, None].expand(T, 3).contiguous()
            cache_pos = tok_d[1].contiguous()
        f = N.RfStackForward()
        f.hidden, f.tokens, f.decode = self.hidden.data_ptr(), T, 0
        f.pos, f.pos_stride = pos_d.data_ptr(), self.pos_stride
        f.cos, f.sin = self.cos.data_ptr(), self.sin.data_ptr()
        f.axis_of_freq = None if self.axis is None else self.axis.data_ptr()
        f.seq_of_tok, f.cache_pos = seq_local.data_ptr(), cache_pos.data_ptr()
        f.num_seqs = n
        qs, ql, kl = meta_d[0].contiguous(), meta_d[1].contiguous(), meta_d[2].contiguous()
        f.q_start, f.q_len, f.kv_len = qs.data_ptr(), ql.data_ptr(), kl.data_ptr()
        f.max_q_len = max(c[2] for c in ch)
        f.max_kv_len = max(starts[c[0]] + c[1] + c[2] for c in ch)
        f.page_table, f.pt_stride, f.pool_pages = pt.data_ptr(), pt.stride(0), self.cache.num_pages
        if self.gdn_layers:
            slot_d, fresh_d = meta_d[3].contiguous(), meta_d[5].contiguous()
            f.state_slot, f.state_fresh = slot_d.data_ptr(), fresh_d.data_ptr()
        if ds_rows:
            ds_rows_d = torch.cat(ds_rows).to(torch.int32).pin_memory().to(self.device, non_blocking=True)
            ds_layers = [torch.cat(parts).contiguous() for parts in ds_feats]
            ds_ptrs = torch.tensor([t.data_ptr() for t in ds_layers], dtype=torch.int64)   # host array of device pointers
            f.deepstack, f.deepstack_rows = ds_ptrs.data_ptr(), ds_rows_d.data_ptr()
            f.n_deepstack, f.n_deepstack_rows = len(ds_layers), ds_rows_d.numel()
        N.check(N.lib().rf_stack_forward(self.handle, C.byref(f), self._stream()), "rf_stack_forward")
        if row_logits is not None:                 # logits of the requested trailing rows of every sequence in this chunk
            keep = row_logits["keep"]
            o2 = 0
            for (s, off, cnt) in ch:
                lo = 0 if keep == 0 else max(lens[s] - keep, 0)
                a, b = max(off, lo), off + cnt
                for r0 in range(a, b, self.max_batch):
                    nr = min(self.max_batch, b - r0)
                    idx = torch.arange(o2 + r0 - off, o2 + r0 - off + nr, dtype=torch.int32, device=self.device)
                    lg = torch.empty((nr, self.vocab_local), dtype=self.dtype, device=self.device)
                    self._head(nr, idx, lg)
                    row_logits["out"][s].append(lg)
                o2 += cnt
        # sequences whose prompt ends in this chunk get their first token
        done = [(j, s) for j, (s, off, cnt) in enumerate(ch) if off + cnt == lens[s]]
        if done:
            rows = meta_d[4][torch.tensor([j for j, _ in done], device=self.device)].contiguous()
            for b0 in range(0, len(done), self.max_batch):
                sub = done[b0:b0 + self.max_batch]
                lg = torch.empty((len(sub), self.vocab_local), dtype=self.dtype, device=self.device) if logits_all is not None else None
                self._head(len(sub), rows[b0:b0 + len(sub)].contiguous(), lg)
                dst = torch.tensor([s for _, s in sub], device=self.device)
                first[dst] = self.out_ids[:len(sub)]
                if logits_all is not None:
                    logits_all[dst] = lg

    # ------------------------------------------------------------------- decode
    def _decode_step(self, B: int, logits_out: Optional[torch.Tensor] = None) -> None:
        self._embed(self.ids[:B], B)
        f = N.RfStackForward()
        f.hidden, f.tokens, f.decode = self.hidden.data_ptr(), B, 1
        f.pos, f.pos_stride = self.pos.data_ptr(), self.pos_stride
        f.cos, f.sin = self.cos.data_ptr(), self.sin.data_ptr()
        f.axis_of_freq = None if self.axis is None else self.axis.data_ptr()
        f.num_seqs = B
        f.kv_len = self.kv_len.data_ptr()
        f.max_q_len, f.max_kv_len = 1, self.max_seq_len
        pt = self.cache.page_table
        f.page_table, f.pt_stride, f.pool_pages = pt.data_ptr(), pt.stride(0), self.cache.num_pages
        N.check(N.lib().rf_stack_forward(self.handle, C.byref(f), self._stream()), "rf_stack_forward")
        self._head(B, None, logits_out)
        N.check(N.lib().rf_decode_advance(C.c_void_p(self.pos.data_ptr()), self.pos_stride,
                                          C.c_void_p(self.kv_len.data_ptr()), B, C.c_void_p(self.out_ids.data_ptr()),
                                          C.c_void_p(self.ids.data_ptr()), C.c_void_p(self.hist.data_ptr()),
                                          C.c_void_p(self.step.data_ptr()), self.hist_steps, self._stream()),
                "rf_decode_advance")

    def capture(self, B: int) -> None:
        """BUILD: run one eager step (loads kernels, sets attributes), rewind, then capture."""
        if B in self.graphs:
            return
        snap = (self.pos.clone(), self.kv_len.clone(), self.ids.clone(), self.step.clone())
        # recurrent layers are not idempotent: the eager build step must not advance their state
        gdn_snap = {l: (self.gdn_conv_state[l].clone(), self.gdn_rec_state[l].clone()) for l in self.gdn_layers}
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._decode_step(B)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            self._decode_step(B)
        torch.cuda.synchronize()
        self.pos.copy_(snap[0]); self.kv_len.copy_(snap[1]); self.ids.copy_(snap[2]); self.step.copy_(snap[3])
        for l, (cv, rc) in gdn_snap.items():
            self.gdn_conv_state[l].copy_(cv)
            self.gdn_rec_state[l].copy_(rc)
        self.graphs[B] = g

    def decode(self, n_steps: int, *, use_graph: bool = True) -> torch.Tensor:
        """Run ``n_steps`` greedy steps for the prefilled batch; returns tokens [B, n_steps] (device).
        The token produced by prefill is NOT included; step i's output is the (i+2)-th new token."""
        B = self.batch
        if B == 0:
            raise RPUBackendError("decode() before prefill()")
        for s in range(B):
            self.cache.check_fits(s, n_steps + 1)
        self._liveness()
        self.reserve_steps(n_steps)
        start = int(self.step.item())
        if start + n_steps > self.hist_steps:
            self.step.zero_()
            start = 0
        if use_graph:
            self.capture(B)
            g = self.graphs[B]
            for _ in range(n_steps):
                g.replay()
        else:
            for _ in range(n_steps):
                self._decode_step(B)
        self.cache.lengths[:B] += n_steps
        return self.hist[start:start + n_steps, :B].t()

    def step_from_host(self, host_ids: torch.Tensor, host_out: torch.Tensor) -> None:
        """One decode step driven from the host: copy this step's input ids from pinned host
        memory, replay the graph, copy the produced ids back (asynchronous; the caller syncs)."""
        B = self.batch
        self._host_steps += 1
        if self.tp.enabled and self.heartbeat_every > 0 and self._host_steps % self.heartbeat_every == 0:
            self._liveness()
        self.cache.ensure_batch(B, 2)            # one vector comparison unless a sequence crosses a page boundary
        self.ids[:B].copy_(host_ids, non_blocking=True)
        self.graphs[B].replay()
        host_out.copy_(self.out_ids[:B], non_blocking=True)
        self.cache.lengths[:B] += 1

    @torch.no_grad()
    def generate(self, prompts: Sequence[torch.Tensor], max_new_tokens: int, *, use_graph: bool = True) -> torch.Tensor:
        first = self.prefill(prompts)
        if max_new_tokens <= 1:
            return first[:, None]
        rest = self.decode(max_new_tokens - 1, use_graph=use_graph)
        out = torch.cat((first[:, None], rest), 1)
        self.check_status()
        return out

    def close(self) -> None:
        lib = N.lib()
        torch.cuda.synchronize()
        self.graphs.clear()
        if self.comm is not None:
            self.comm.close()
            self.comm = None
        if getattr(self, "handle", None) is not None:
            lib.rf_stack_destroy(self.handle)
            self.handle = None
        if getattr(self, "cache", None) is not None:
            self.cache.close()
