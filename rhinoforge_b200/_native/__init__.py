"""ctypes binding of ``librf_b200.so`` (the sm_100a kernel + runtime library).

The library is built in-tree by :mod:`rhinoforge_b200.csrc.build` and loaded
lazily: importing the package never touches it, host-only code paths
(planners, registries) work without it, and anything that needs a kernel
raises :class:`NativeLibraryError` if it is missing instead of silently
falling back to PyTorch.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "librf_b200.so"

_lock = threading.Lock()
_lib: C.CDLL | None = None


class NativeLibraryError(RuntimeError):
    """librf_b200.so is missing or a native call failed."""


class RfGemm(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("ldx", C.c_int64),
        ("w", C.c_void_p), ("ldw", C.c_int64),
        ("out", C.c_void_p), ("ldo", C.c_int64),
        ("residual", C.c_void_p), ("ldr", C.c_int64),
        ("bias", C.c_void_p), ("scale", C.c_void_p), ("row_scale", C.c_void_p),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("dtype", C.c_int32), ("act", C.c_int32), ("dual_offset", C.c_int32), ("w_int8", C.c_int32),
        ("ws", C.c_void_p), ("ws_bytes", C.c_uint64),
        ("sem", C.c_void_p), ("sem_count", C.c_int32),
        ("status", C.c_void_p),
        ("ar_world", C.c_int32), ("ar_rank", C.c_int32),
        ("ar_recv", C.c_void_p), ("ar_flags", C.c_void_p), ("ar_state", C.c_void_p),
        ("ar_recv_bytes", C.c_uint64), ("ar_flag_count", C.c_int32),
        ("force_splits", C.c_int32), ("force_swap", C.c_int32), ("force_bn", C.c_int32), ("w_packed", C.c_int32),
        ("w_scratch", C.c_void_p), ("w_scratch_bytes", C.c_uint64),
        ("ar_publish", C.c_int32), ("ar_cnt_base", C.c_int32),
        ("prefetch", C.c_void_p), ("prefetch_bytes", C.c_uint64),
        ("w_bits", C.c_int32), ("w_group", C.c_int32), ("w_fp4", C.c_int32), ("ss_tiles", C.c_int32),
        ("ss_out", C.c_void_p), ("ss_in", C.c_void_p), ("ss_ld", C.c_int32), ("ss_dim", C.c_int32),
        ("ss_eps", C.c_float), ("streaming_only", C.c_int32),
    ]


class RfArConsume(C.Structure):
    _fields_ = [
        ("M", C.c_int32), ("N", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32),
        ("ar_recv", C.c_void_p), ("ar_flags", C.c_void_p), ("ar_state", C.c_void_p),
        ("ar_recv_bytes", C.c_uint64), ("ar_cnt_base", C.c_int32), ("pub_ctas", C.c_int32),
        ("residual", C.c_void_p), ("ldr", C.c_int64), ("out", C.c_void_p), ("ldo", C.c_int64),
        ("norm_w", C.c_void_p), ("norm_out", C.c_void_p), ("ldn", C.c_int64),
        ("eps", C.c_float), ("norm_mode", C.c_int32), ("status", C.c_void_p), ("dtype", C.c_int32),
    ]


class RfMoeGroupedGemm(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("ldx", C.c_int64), ("w", C.c_void_p), ("out", C.c_void_p), ("ldo", C.c_int64),
        ("row_scale", C.c_void_p), ("tiles", C.c_void_p),
        ("max_rows", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("dual", C.c_int32), ("act", C.c_int32),
        ("bank_section_row_tiles", C.c_int32), ("bank_kb_total", C.c_int32),
        ("rt_per_expert", C.c_int32), ("kb_per_expert", C.c_int32), ("dtype", C.c_int32), ("status", C.c_void_p),
    ]


class RfRopeKv(C.Structure):
    _fields_ = [
        ("qkv", C.c_void_p), ("ld", C.c_int64),
        ("q_out", C.c_void_p), ("ldq", C.c_int64),
        ("tokens", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("hd", C.c_int32), ("rot_dim", C.c_int32),
        ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p),
        ("eps", C.c_float), ("norm_mode", C.c_int32),
        ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("pos", C.c_void_p), ("pos_stride", C.c_int32),
        ("axis_of_freq", C.c_void_p),
        ("k_pool", C.c_void_p), ("v_pool", C.c_void_p),
        ("page_table", C.c_void_p), ("pt_stride", C.c_int32),
        ("seq_of_tok", C.c_void_p), ("cache_pos", C.c_void_p),
        ("rope_before_norm", C.c_int32), ("write_k_inplace", C.c_int32), ("dtype", C.c_int32),
        ("v_norm", C.c_int32),
    ]


class RfAttn(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("ldq", C.c_int64),
        ("out", C.c_void_p), ("ldo", C.c_int64),
        ("q_rows_total", C.c_int64),
        ("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("pool_pages", C.c_int64),
        ("page_table", C.c_void_p), ("pt_stride", C.c_int32),
        ("k", C.c_void_p), ("v", C.c_void_p), ("ldk", C.c_int64), ("ldv", C.c_int64), ("kv_rows_total", C.c_int64),
        ("num_seqs", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("hd", C.c_int32),
        ("q_start", C.c_void_p), ("q_len", C.c_void_p), ("kv_start", C.c_void_p), ("kv_len", C.c_void_p),
        ("max_q_len", C.c_int32), ("max_kv_len", C.c_int32),
        ("causal", C.c_int32), ("window", C.c_int32),
        ("mask", C.c_void_p), ("mask_ld", C.c_int64), ("mask_seq_stride", C.c_int64),
        ("seg_q", C.c_void_p), ("seg_k", C.c_void_p),
        ("scale", C.c_float),
        ("ws", C.c_void_p), ("ws_bytes", C.c_uint64),
        ("status", C.c_void_p), ("dtype", C.c_int32),
    ]


class RfStackConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("layers", "hidden", "Hq", "Hkv", "hd", "inter", "rot_dim", "norm_kind",
                                         "mlp_kind")] + [("eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("qk_norm", "rope_before_norm", "gated_residual", "sandwich_norm", "paged_kv",
                                         "causal", "window")] + [("attn_scale", C.c_float)] + \
               [(n, C.c_int32) for n in ("true_hd", "dtype", "max_tokens", "max_seqs", "vocab_local", "vocab_offset",
                                         "tp_world", "tp_rank", "weights_int8", "decode_gemv_max_m", "attn_gate",
                                         "gdn_Hk", "gdn_Hv", "gdn_Dk", "gdn_Dv", "gdn_conv_k", "weights_packed",
                                         "moe_experts", "moe_top_k", "moe_expert_inter", "moe_score_fn",
                                         "moe_norm_topk")] + [("moe_routed_scale", C.c_float)] + \
               [("weights_bits", C.c_int32), ("weights_group", C.c_int32), ("norm_folded", C.c_int32),
                ("gemm_streaming_only", C.c_int32)]


class RfLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "norm1_w", "norm1_b", "wqkv", "bqkv", "sqkv", "q_norm_w", "k_norm_w", "wo", "bo", "so", "norm2_w", "norm2_b",
        "w_up", "b_up", "s_up", "w_down", "b_down", "s_down", "post_attn_norm_w", "post_mlp_norm_w", "k_pool",
        "v_pool")] + [("mixer", C.c_int64)] + [(n, C.c_void_p) for n in (
        "gdn_conv_w", "gdn_A_log", "gdn_dt_bias", "gdn_norm_w", "gdn_conv_state", "gdn_rec_state",
        "moe_router_w", "moe_router_bias")]


class RfStackComm(C.Structure):
    _fields_ = [("recv", C.c_void_p), ("flags", C.c_void_p), ("state", C.c_void_p),
                ("recv_half_bytes", C.c_uint64), ("flag_count", C.c_int32), ("cnt_base", C.c_int32),
                ("sym_rows", C.c_int32), ("rows_flag_base", C.c_int32),
                ("sym_hidden", C.c_void_p), ("sym_xn", C.c_void_p), ("sym_tmp", C.c_void_p), ("sym_partial", C.c_void_p),
                ("hidden_tab", C.c_void_p), ("xn_tab", C.c_void_p), ("tmp_tab", C.c_void_p), ("partial_tab", C.c_void_p)]


class RfArRows(C.Structure):
    _fields_ = [
        ("M", C.c_int32), ("N", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32),
        ("partial_tab", C.c_void_p), ("out_tab", C.c_void_p), ("norm_tab", C.c_void_p), ("ar_flags", C.c_void_p),
        ("ar_state", C.c_void_p), ("flag_base", C.c_int32), ("add_residual", C.c_int32),
        ("norm_w", C.c_void_p), ("eps", C.c_float), ("norm_mode", C.c_int32), ("status", C.c_void_p), ("dtype", C.c_int32),
        ("out_local", C.c_int32),
    ]


class RfStackForward(C.Structure):
    _fields_ = [
        ("hidden", C.c_void_p), ("tokens", C.c_int32), ("decode", C.c_int32),
        ("pos", C.c_void_p), ("pos_stride", C.c_int32),
        ("cos", C.c_void_p), ("sin", C.c_void_p), ("axis_of_freq", C.c_void_p),
        ("seq_of_tok", C.c_void_p), ("cache_pos", C.c_void_p),
        ("num_seqs", C.c_int32),
        ("q_start", C.c_void_p), ("q_len", C.c_void_p), ("kv_start", C.c_void_p), ("kv_len", C.c_void_p),
        ("max_q_len", C.c_int32), ("max_kv_len", C.c_int32),
        ("page_table", C.c_void_p), ("pt_stride", C.c_int32), ("pool_pages", C.c_int64),
        ("mask", C.c_void_p), ("mask_ld", C.c_int64), ("mask_seq_stride", C.c_int64),
        ("seg_q", C.c_void_p), ("seg_k", C.c_void_p),
        ("mod", C.c_void_p), ("rows_per_mod", C.c_int32),
        ("layer_begin", C.c_int32), ("layer_end", C.c_int32),
        ("deepstack", C.c_void_p), ("deepstack_rows", C.c_void_p), ("n_deepstack", C.c_int32),
        ("n_deepstack_rows", C.c_int32),
        ("taps", C.c_void_p), ("tap_layers", C.c_void_p), ("n_taps", C.c_int32),
        ("state_slot", C.c_void_p), ("state_fresh", C.c_void_p),
        ("twin_split", C.c_int32), ("reserved0", C.c_int32),
    ]


class RfConv1d(C.Structure):
    _fields_ = [("x", C.c_void_p), ("ldx", C.c_int64), ("y", C.c_void_p), ("ldy", C.c_int64), ("w", C.c_void_p),
                ("state", C.c_void_p), ("q_start", C.c_void_p), ("q_len", C.c_void_p), ("slot", C.c_void_p)] + \
               [(n, C.c_int32) for n in ("num_seqs", "max_q_len", "C", "K", "silu", "dtype")]


class RfGdn(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("ld", C.c_int64), ("b", C.c_void_p), ("a", C.c_void_p), ("ld_ba", C.c_int64),
                ("out", C.c_void_p), ("ldo", C.c_int64), ("state", C.c_void_p), ("A_log", C.c_void_p),
                ("dt_bias", C.c_void_p), ("q_start", C.c_void_p), ("q_len", C.c_void_p), ("slot", C.c_void_p),
                ("fresh", C.c_void_p)] + [(n, C.c_int32) for n in ("num_seqs", "Hk", "Hv", "Dk", "Dv", "dtype")]


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    """Return the loaded library, building it first when nvcc is present."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            if os.environ.get("RF_B200_NO_BUILD") == "1":
                raise NativeLibraryError(f"{LIB_PATH} not found and RF_B200_NO_BUILD=1")
            try:
                from ..csrc.build import build
                build()
            except Exception as e:  # noqa: BLE001
                raise NativeLibraryError(f"{LIB_PATH} not found and building it failed: {e}") from e
        l = C.CDLL(str(LIB_PATH))
        l.rf_last_error.restype = C.c_char_p
        l.rf_argmax_scratch_bytes.restype = C.c_uint64
        l.rf_attn_decode_scratch_bytes.restype = C.c_uint64
        l.rf_stack_create.restype = C.c_int64
        l.rf_stack_arena_bytes.restype = C.c_uint64
        l.rf_stack_status_ptr.restype = C.c_void_p
        l.rf_kvpool_create.restype = C.c_int64
        l.rf_pack_weight_bytes.restype = C.c_uint64
        l.rf_pack_w4_bytes.restype = C.c_uint64
        l.rf_pack_w4_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int32, C.c_int32]
        for fn in ("rf_stack_destroy", "rf_stack_set_layer", "rf_stack_set_head", "rf_stack_set_comm",
                   "rf_stack_arena_bytes", "rf_stack_bind_arena", "rf_stack_status_ptr", "rf_stack_forward",
                   "rf_stack_head", "rf_stack_final_norm", "rf_kvpool_destroy", "rf_kvpool_reserve",
                   "rf_kvpool_release", "rf_kvpool_free_pages"):
            getattr(l, fn).argtypes = None
        _lib = l
    return _lib


def check(rc: int, what: str = "native call") -> None:
    if rc != 0:
        msg = lib().rf_last_error().decode(errors="replace")
        from ..api.errors import RPUBackendError
        raise RPUBackendError(f"{what} failed ({rc}): {msg}")
