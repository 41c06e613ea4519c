"""Paged KV pool: ``[layers, 2, pages, kv_heads, 16, head_dim]`` device memory plus a page table.

One page holds 16 tokens of every local KV head -- the same contiguous 16-token slab the
reference's blocked cache uses (``python/rpu_backend/api/cache.py:78-197``), addressed through a
page table instead of a fixed 7-D view.  Page ownership is kept by the native ``KvPool``
(``csrc/runtime/kv_pool.cpp``); ``position`` per sequence is host state and the only source of
truth for lengths.  The pool is zero-filled at creation and must never hold NaN/Inf: masked
tokens still pass through the attention MMAs.

Pages are handed out ON DEMAND: a sequence owns only the pages its tokens (plus the step about to
run) need, ``ensure(seq, tokens)`` grows it, ``release(seq)`` returns its pages.  The pool may
therefore be smaller than ``batch_size * max_seq_len`` (``pool_tokens``): short sequences leave room
for long ones, and a request the pool cannot serve raises ``SPMExhaustionError`` before anything
runs.  Because sequences grow interleaved, the page table is in general not the identity map.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from .. import _native as N
from .errors import RPUBackendError

PAGE_TOKENS = 16


class PagedKV:
    def __init__(self, num_layers: int, batch_size: int, max_seq_len: int, num_kv_heads: int, head_dim: int, *,
                 device="cuda", dtype=torch.float16, pool_tokens: Optional[int] = None):
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
        if pool_tokens is not None:
            if isinstance(pool_tokens, bool) or not isinstance(pool_tokens, int) or pool_tokens <= 0:
                raise ValueError(f"RPUCache pool_tokens must be a positive integer, got {pool_tokens!r}")
            self.num_pages = min(self.num_pages, (pool_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS)
        self.kv = torch.zeros((num_layers, 2, self.num_pages, num_kv_heads, PAGE_TOKENS, head_dim), dtype=dtype,
                              device=self.device)
        self.page_table = torch.zeros((batch_size, self.pages_per_seq), dtype=torch.int32, device=self.device)
        self._pt_host = torch.zeros((batch_size, self.pages_per_seq), dtype=torch.int32)
        if self.device.type == "cuda":
            self._pt_host = self._pt_host.pin_memory()
        # cached length and page capacity (in tokens) of every sequence slot: numpy so that a decode step
        # advances / checks the whole batch with one vector operation
        self.lengths = np.zeros(batch_size, dtype=np.int64)
        self._capacity = np.zeros(batch_size, dtype=np.int64)
        self._dirty = False
        self._pool = None
        if N.available() or self.device.type == "cuda":
            self._pool = C.c_int64(N.lib().rf_kvpool_create(self.num_pages, batch_size, self.pages_per_seq))
        else:  # host-only sizing without the native library: identity mapping
            if self.num_pages < batch_size * self.pages_per_seq:
                raise ValueError("an over-subscribed pool (pool_tokens) needs the native library")
            for s in range(batch_size):
                self._pt_host[s] = torch.arange(s * self.pages_per_seq, (s + 1) * self.pages_per_seq)
            self._capacity[:] = self.pages_per_seq * PAGE_TOKENS

    # -- page ownership ----------------------------------------------------------------------
    def ensure(self, seq: int, tokens: int) -> bool:
        """Grow sequence ``seq`` until it owns pages for ``tokens`` tokens; True when pages were added (the device
        table is then stale until :meth:`sync_table`).  Raises ``SPMExhaustionError`` when the pool has no free
        page left or ``tokens`` exceeds ``max_seq_len``; nothing is changed then."""
        if tokens <= self._capacity[seq]:
            return False
        if self._pool is None:
            raise RPUBackendError(f"sequence {seq} needs {tokens} tokens, the host-only cache holds {self._capacity[seq]}")
        row = self._pt_host[seq]
        rc = N.lib().rf_kvpool_reserve(self._pool, seq, int(tokens), C.c_void_p(row.data_ptr()))
        if rc != 0:
            from ..api.errors import SPMExhaustionError
            raise SPMExhaustionError(N.lib().rf_last_error().decode(errors="replace"))
        self._capacity[seq] = (int(tokens) + PAGE_TOKENS - 1) // PAGE_TOKENS * PAGE_TOKENS
        self._dirty = True
        return True

    def ensure_batch(self, n_seqs: int, extra: int) -> None:
        """Every sequence ``0..n_seqs-1`` gets room for ``extra`` more tokens; the device table is refreshed when
        a page was added.  The common case (room is there) costs one vector comparison."""
        need = self.lengths[:n_seqs] + extra
        short = np.nonzero(need > self._capacity[:n_seqs])[0]
        for s in short:
            self.ensure(int(s), int(need[s]))
        if self._dirty:
            self.sync_table()

    def reserve(self, seq: int, tokens: Optional[int] = None) -> None:
        """Give sequence ``seq`` pages for ``tokens`` tokens up front (default: the full ``max_seq_len``)."""
        self.ensure(seq, self.max_seq_len if tokens is None else tokens)

    def reserve_all(self) -> None:
        """Reserve ``max_seq_len`` for every slot up front (the fixed-envelope behaviour; needs a full-size pool)."""
        for s in range(self.batch_size):
            self.reserve(s)
        self.sync_table()

    def sync_table(self) -> None:
        self.page_table.copy_(self._pt_host, non_blocking=True)
        self._dirty = False

    def release(self, seq: int) -> None:
        if self._pool is not None:
            N.lib().rf_kvpool_release(self._pool, seq)
            self._capacity[seq] = 0
            self._pt_host[seq].zero_()
            self._dirty = True
        self.lengths[seq] = 0

    def owned_pages(self, seq: int) -> int:
        return int(self._capacity[seq]) // PAGE_TOKENS

    def free_pages(self) -> int:
        return N.lib().rf_kvpool_free_pages(self._pool) if self._pool is not None else 0

    def layer_ptrs(self, layer: int):
        return self.kv[layer, 0].data_ptr(), self.kv[layer, 1].data_ptr()

    # -- contents ------------------------------------------------------------------------------
    def gather(self, layer: int, seq: int, length: Optional[int] = None):
        """Dense ``(K, V)`` of one sequence: ``[kv_heads, length, head_dim]`` each."""
        L = int(self.lengths[seq] if length is None else length)
        npg = (L + PAGE_TOKENS - 1) // PAGE_TOKENS
        pages = self._pt_host[seq, :npg].long().to(self.device)
        k = self.kv[layer, 0][pages]  # [npg, H, 16, hd]
        v = self.kv[layer, 1][pages]
        k = k.permute(1, 0, 2, 3).reshape(self.num_kv_heads, npg * PAGE_TOKENS, self.head_dim)[:, :L]
        v = v.permute(1, 0, 2, 3).reshape(self.num_kv_heads, npg * PAGE_TOKENS, self.head_dim)[:, :L]
        return k, v

    def scatter(self, layer: int, seq: int, k: torch.Tensor, v: torch.Tensor, start: int = 0) -> None:
        """Write dense ``k, v [kv_heads, L, head_dim]`` (already rotated) into rows ``[start, start + L)`` of one
        sequence's pages: the inverse of :meth:`gather` (keys and values computed elsewhere, e.g. a prefix that another
        model produced).  The pages must be owned already (:meth:`ensure`); ``lengths`` is left to the caller."""
        L = int(k.shape[1])
        if tuple(k.shape) != (self.num_kv_heads, L, self.head_dim) or tuple(v.shape) != tuple(k.shape):
            raise ValueError(f"expected [kv_heads={self.num_kv_heads}, L, head_dim={self.head_dim}], got {tuple(k.shape)} / "
                             f"{tuple(v.shape)}")
        if start + L > int(self._capacity[seq]):
            raise ValueError(f"rows [{start}, {start + L}) exceed the {int(self._capacity[seq])} rows sequence {seq} owns")
        rows = torch.arange(start, start + L)
        pages = self._pt_host[seq][(rows // PAGE_TOKENS).long()].long().to(self.device)
        slot = (rows % PAGE_TOKENS).to(self.device)
        for idx, t in ((0, k), (1, v)):
            self.kv[layer, idx][pages, :, slot] = t.to(self.device, self.dtype).transpose(0, 1)

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
