"""Paged KV pool: ``[layers, 2, pages, kv_heads, 16, head_dim]`` device memory plus a page table.

One page holds 16 tokens of every local KV head -- the same contiguous 16-token slab the
reference's blocked cache uses (``python/rpu_backend/api/cache.py:78-197``), addressed through a
page table instead of a fixed 7-D view.  Page ownership is kept by the native ``KvPool``
(``csrc/runtime/kv_pool.cpp``); ``position`` per sequence is host state and the only source of
truth for lengths.  The pool is zero-filled at creation and must never hold NaN/Inf: masked
tokens still pass through the attention MMAs.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from .. import _native as N
from .errors import RPUBackendError

PAGE_TOKENS = 16


class PagedKV:
    def __init__(self, num_layers: int, batch_size: int, max_seq_len: int, num_kv_heads: int, head_dim: int, *,
                 device="cuda", dtype=torch.float16):
        for name, v in (("num_layers", num_layers), ("batch_size", batch_size), ("max_seq_len", max_seq_len),
                        ("num_kv_heads", num_kv_heads), ("head_dim", head_dim)):
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ValueError(f"RPUCache {name} must be a positive integer, got {v!r}")
        if head_dim % 16:
            raise ValueError(f"RPUCache head_dim must be divisible by 16, got {head_dim}")
        self._pool = None
        self.num_layers, self.batch_size, self.max_seq_len = num_layers, batch_size, max_seq_len
        self.num_kv_heads, self.head_dim, self.dtype = num_kv_heads, head_dim, dtype
        self.device = torch.device(device)
        self.pages_per_seq = (max_seq_len + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.num_pages = batch_size * self.pages_per_seq
        self.kv = torch.zeros((num_layers, 2, self.num_pages, num_kv_heads, PAGE_TOKENS, head_dim), dtype=dtype,
                              device=self.device)
        self.page_table = torch.zeros((batch_size, self.pages_per_seq), dtype=torch.int32, device=self.device)
        self._pt_host = torch.zeros((batch_size, self.pages_per_seq), dtype=torch.int32)
        if self.device.type == "cuda":
            self._pt_host = self._pt_host.pin_memory()
        self.lengths: List[int] = [0] * batch_size
        self._pool = None
        if N.available() or self.device.type == "cuda":
            self._pool = C.c_int64(N.lib().rf_kvpool_create(self.num_pages, batch_size, self.pages_per_seq))
        else:  # host-only sizing without the native library: identity mapping
            for s in range(batch_size):
                self._pt_host[s] = torch.arange(s * self.pages_per_seq, (s + 1) * self.pages_per_seq)
        self._reserved = [False] * batch_size

    # -- page ownership ----------------------------------------------------------------------
    def reserve(self, seq: int, tokens: Optional[int] = None) -> None:
        """Give sequence ``seq`` pages for ``tokens`` tokens (default: the full ``max_seq_len``)."""
        tokens = self.max_seq_len if tokens is None else tokens
        if self._pool is None:
            self._reserved[seq] = True
            return
        row = self._pt_host[seq]
        rc = N.lib().rf_kvpool_reserve(self._pool, seq, tokens, C.c_void_p(row.data_ptr()))
        if rc != 0:
            from ..api.errors import SPMExhaustionError
            raise SPMExhaustionError(N.lib().rf_last_error().decode(errors="replace"))
        self._reserved[seq] = True

    def reserve_all(self) -> None:
        for s in range(self.batch_size):
            if not self._reserved[s]:
                self.reserve(s)
        self.sync_table()

    def sync_table(self) -> None:
        self.page_table.copy_(self._pt_host, non_blocking=True)

    def release(self, seq: int) -> None:
        if self._pool is not None:
            N.lib().rf_kvpool_release(self._pool, seq)
        self._reserved[seq] = False
        self.lengths[seq] = 0

    def free_pages(self) -> int:
        return N.lib().rf_kvpool_free_pages(self._pool) if self._pool is not None else 0

    def layer_ptrs(self, layer: int):
        return self.kv[layer, 0].data_ptr(), self.kv[layer, 1].data_ptr()

    # -- contents ------------------------------------------------------------------------------
    def gather(self, layer: int, seq: int, length: Optional[int] = None):
        """Dense ``(K, V)`` of one sequence: ``[kv_heads, length, head_dim]`` each."""
        L = self.lengths[seq] if length is None else length
        npg = (L + PAGE_TOKENS - 1) // PAGE_TOKENS
        pages = self._pt_host[seq, :npg].long().to(self.device)
        k = self.kv[layer, 0][pages]  # [npg, H, 16, hd]
        v = self.kv[layer, 1][pages]
        k = k.permute(1, 0, 2, 3).reshape(self.num_kv_heads, npg * PAGE_TOKENS, self.head_dim)[:, :L]
        v = v.permute(1, 0, 2, 3).reshape(self.num_kv_heads, npg * PAGE_TOKENS, self.head_dim)[:, :L]
        return k, v

    def zero_(self) -> None:
        self.kv.zero_()

    def close(self) -> None:
        if getattr(self, "_pool", None) is not None:
            try:
                N.lib().rf_kvpool_destroy(self._pool)
            except Exception:  # noqa: BLE001
                pass
            self._pool = None

    def __del__(self):
        self.close()

    def nbytes(self) -> int:
        return self.kv.numel() * self.kv.element_size()

    def check_fits(self, seq: int, extra: int) -> None:
        if self.lengths[seq] + extra > self.max_seq_len:
            raise RPUBackendError(f"RPUCache position overflow: position={self.lengths[seq]}, seq_len={extra}, "
                                  f"max_seq_len={self.max_seq_len}")
