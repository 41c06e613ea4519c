"""Tensor-parallel context: one process per GPU, ``torch.distributed`` for the
rendezvous, CUDA-IPC peer buffers for the fused GEMM+all-reduce kernels.

The reference's only parallelism is 8-way tensor parallelism over the cores of
one chip (column-partitioned q/k/v/gate/up/lm_head, row-partitioned
o_proj/down_proj followed by all-reduce + residual:
``python/rpu_backend/runtime/weights.py:97-135``, ``src/fused/rpu_qwen3_model.h:3517-3536``).
Here the same rule shards a model over 1/2/4/8 B200s; the all-reduce runs inside
the producing GEMM kernel over NVLink peer stores.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as N
from .. import _native as N_    # the same module under a name that an argument called N cannot shadow


@dataclass
class TPContext:
    rank: int = 0
    world: int = 1
    group: object = None
    device: Optional[torch.device] = None

    @property
    def enabled(self) -> bool:
        return self.world > 1

    @classmethod
    def single(cls, device=None) -> "TPContext":
        return cls(0, 1, None, torch.device(device) if device is not None else None)

    @classmethod
    def from_env(cls, backend: Optional[str] = None) -> "TPContext":
        """Join the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* (torchrun)."""
        import torch.distributed as dist
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world == 1:
            dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
            return cls(0, 1, None, dev)
        rank = int(os.environ["RANK"])
        local = int(os.environ.get("LOCAL_RANK", rank))
        use_cuda = torch.cuda.is_available()
        if use_cuda:
            torch.cuda.set_device(local)
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            kw = {}
            if use_cuda:
                kw["device_id"] = torch.device("cuda", local)
            dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=world, **kw)
        return cls(rank, world, dist.group.WORLD, torch.device("cuda", local) if use_cuda else torch.device("cpu"))

    def barrier(self) -> None:
        if self.enabled:
            import torch.distributed as dist
            dist.barrier(self.group)

    def all_gather_object(self, obj):
        if not self.enabled:
            return [obj]
        import torch.distributed as dist
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def max_float(self, v: float) -> float:
        return max(self.all_gather_object(float(v)))

    # -- host-side liveness ----------------------------------------------------------------------
    # The fused kernels wait on flags that peers write; a peer that died would make every such wait
    # run into its time limit.  Ranks therefore publish a heartbeat in the rendezvous store between
    # steps, and check their peers' heartbeats BEFORE launching the next step: a missing rank is
    # reported on the host, with no kernel in flight.
    def _store(self):
        import torch.distributed as dist
        return dist.distributed_c10d._get_default_store()

    def heartbeat(self, step: int) -> None:
        """Publish "this rank has finished step ``step`` and is still alive"."""
        if self.enabled:
            self._store().set(f"rf_hb/{self.rank}", str(int(step)))

    def check_peers(self, step: int, timeout_s: float = 5.0) -> None:
        """Raise unless every rank has published a heartbeat for ``step`` (or later) within ``timeout_s``."""
        if not self.enabled:
            return
        import time
        from ..runtime.errors import RPUBackendError
        store, deadline = self._store(), time.monotonic() + timeout_s
        missing = list(range(self.world))
        while missing:
            still = []
            for r in missing:
                try:
                    ok = store.check([f"rf_hb/{r}"]) and int(store.get(f"rf_hb/{r}")) >= step
                except Exception:  # noqa: BLE001  (store gone: the rank hosting it died)
                    ok = False
                if not ok:
                    still.append(r)
            missing = still
            if missing and time.monotonic() > deadline:
                raise RPUBackendError(f"tensor-parallel rank(s) {missing} published no heartbeat for step {step} within "
                                      f"{timeout_s:.1f} s; not launching (peer dead or hung)")
            if missing:
                time.sleep(0.01)


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of an even split; ``total`` must divide."""
    if total % world:
        raise ValueError(f"{total} does not split evenly over {world} ranks")
    per = total // world
    return rank * per, (rank + 1) * per


def kv_head_range(num_kv_heads: int, world: int, rank: int) -> tuple[int, int]:
    """KV heads a rank owns: an even split, or one replicated head when ``kv < world``
    (the reference replicates KV heads the same way, ``adapters/pi05/__init__.py:923-946``)."""
    if num_kv_heads >= world:
        return shard_range(num_kv_heads, world, rank)
    if world % num_kv_heads:
        raise ValueError(f"{world} ranks cannot replicate {num_kv_heads} kv heads evenly")
    h = rank // (world // num_kv_heads)
    return h, h + 1


class CommBuffers:
    """Symmetric receive buffer + flag array on every rank, peer-mapped through CUDA IPC.

    Layout of each rank's allocation: ``[recv half 0 | recv half 1 | flags | state]``.
    ``fill(gemm_args)`` wires the pointers into an ``RfGemm`` block.
    """

    FLAG_COUNT = 1 << 20
    BARRIER_FLAGS = 64  # the last flags are reserved: barrier [0, 8), arg-max merge [16, 24), arrival counters [32, 40),
    #                     row all-reduce [40, 56)
    CNT_OFFSET = 32     # arrival counters of the publish / consume all-reduce, one per source rank
    ROWS_OFFSET = 40    # "partial ready" and "rows written" flags of the row all-reduce, eight each
    SYM_NAMES = ("hidden", "xn", "tmp", "partial")
    AUX_ROWS = 1024     # rows of (value, id) pairs per rank in the aux area

    def __init__(self, tp: TPContext, recv_half_bytes: int, *, sym_rows: int = 0, sym_cols: int = 0, sym_elem_bytes: int = 2):
        """``sym_rows`` / ``sym_cols`` > 0 additionally lays out four symmetric ``[sym_rows, sym_cols]`` activation
        buffers (residual stream, normalised rows, side result, GEMM partial) behind the flags: every rank has them at
        the same offsets, so a rank can load the rows it owns from every peer's partial and store finished rows into
        every peer's buffers (the prefill-sized all-reduce)."""
        assert tp.enabled
        self.tp = tp
        lib = N.lib()
        self.recv_half_bytes = (recv_half_bytes + 1023) // 1024 * 1024
        self.flag_bytes = self.FLAG_COUNT * 4
        self.aux_bytes = 2 * 8 * self.AUX_ROWS * 8
        self.sym_rows, self.sym_cols, self.sym_elem_bytes = sym_rows, sym_cols, sym_elem_bytes
        self.sym_bytes = (sym_rows * sym_cols * sym_elem_bytes + 1023) // 1024 * 1024
        self.sym_off = 2 * self.recv_half_bytes + self.flag_bytes + 1024 + self.aux_bytes
        self.total = self.sym_off + len(self.SYM_NAMES) * self.sym_bytes
        p = C.c_void_p()
        N.check(lib.rf_comm_alloc(C.c_uint64(self.total), C.byref(p)), "rf_comm_alloc")
        self.local = p.value
        handle = (C.c_uint8 * 64)()
        N.check(lib.rf_ipc_export(C.c_void_p(self.local), handle), "rf_ipc_export")
        handles = tp.all_gather_object(bytes(handle))
        self.peers: list[int] = []
        self._opened: list[int] = []
        for r, hb in enumerate(handles):
            if r == tp.rank:
                self.peers.append(self.local)
                continue
            buf = (C.c_uint8 * 64).from_buffer_copy(hb)
            q = C.c_void_p()
            N.check(lib.rf_ipc_import(buf, C.byref(q)), "rf_ipc_import")
            self.peers.append(q.value)
            self._opened.append(q.value)
        dev = tp.device
        flag_off = 2 * self.recv_half_bytes
        self.recv_ptrs = torch.tensor(self.peers, dtype=torch.int64, device=dev)
        self.flag_ptrs = torch.tensor([b + flag_off for b in self.peers], dtype=torch.int64, device=dev)
        self.state_ptr = self.local + flag_off + self.flag_bytes
        aux_off = flag_off + self.flag_bytes + 1024
        self.aux_ptrs = torch.tensor([b + aux_off for b in self.peers], dtype=torch.int64, device=dev)
        self.status = torch.zeros(8, dtype=torch.int32, device=dev)
        self.sym_tabs = {}
        if self.sym_bytes:
            for i, name in enumerate(self.SYM_NAMES):
                self.sym_tabs[name] = torch.tensor([b + self.sym_off + i * self.sym_bytes for b in self.peers],
                                                   dtype=torch.int64, device=dev)
        tp.barrier()

    def sym_ptr(self, name: str) -> int:
        """Device address of this rank's symmetric buffer ``name`` (``hidden``, ``xn``, ``tmp`` or ``partial``)."""
        return self.local + self.sym_off + self.SYM_NAMES.index(name) * self.sym_bytes

    def sym_tensor(self, name: str, dtype: torch.dtype) -> torch.Tensor:
        """This rank's symmetric buffer ``name`` as a ``[sym_rows, sym_cols]`` tensor over the communication region
        (no copy; the region outlives the tensor only as long as this object is open)."""
        class _Raw:
            pass
        raw = _Raw()
        typestr = {torch.float16: "<f2", torch.bfloat16: "<u2", torch.float32: "<f4"}[dtype]
        raw.__cuda_array_interface__ = {"shape": (self.sym_rows, self.sym_cols), "typestr": typestr,
                                        "data": (self.sym_ptr(name), False), "version": 2}
        t = torch.as_tensor(raw, device=self.tp.device)
        return t.view(dtype) if dtype == torch.bfloat16 else t

    def fill(self, g) -> None:
        g.ar_world, g.ar_rank = self.tp.world, self.tp.rank
        g.ar_recv, g.ar_flags = self.recv_ptrs.data_ptr(), self.flag_ptrs.data_ptr()
        g.ar_state = self.state_ptr
        g.ar_recv_bytes = self.recv_half_bytes
        g.ar_flag_count = self.FLAG_COUNT - self.BARRIER_FLAGS
        g.ar_cnt_base = self.cnt_base

    def stack_comm(self) -> "N.RfStackComm":
        c = N.RfStackComm()
        c.recv, c.flags, c.state = self.recv_ptrs.data_ptr(), self.flag_ptrs.data_ptr(), self.state_ptr
        c.recv_half_bytes = self.recv_half_bytes
        c.flag_count = self.FLAG_COUNT - self.BARRIER_FLAGS
        c.cnt_base = self.cnt_base
        if self.sym_bytes:
            c.sym_rows = self.sym_rows
            c.rows_flag_base = self.FLAG_COUNT - self.BARRIER_FLAGS + self.ROWS_OFFSET
            c.sym_hidden, c.sym_xn = self.sym_ptr("hidden"), self.sym_ptr("xn")
            c.sym_tmp, c.sym_partial = self.sym_ptr("tmp"), self.sym_ptr("partial")
            c.hidden_tab, c.xn_tab = self.sym_tabs["hidden"].data_ptr(), self.sym_tabs["xn"].data_ptr()
            c.tmp_tab, c.partial_tab = self.sym_tabs["tmp"].data_ptr(), self.sym_tabs["partial"].data_ptr()
        return c

    @property
    def cnt_base(self) -> int:
        return self.FLAG_COUNT - self.BARRIER_FLAGS + self.CNT_OFFSET

    def consume_args(self, M: int, N: int, pub_ctas: int, out: torch.Tensor, residual=None, norm_w=None,
                     norm_out=None, eps: float = 1e-6, norm_mode: int = 0, status=None) -> "N.RfArConsume":
        """Argument block of ``rf_ar_consume`` for a GEMM launched with ``ar_publish`` on these buffers."""
        a = N_.RfArConsume()
        a.M, a.N, a.world, a.rank = M, N, self.tp.world, self.tp.rank
        a.ar_recv, a.ar_flags, a.ar_state = self.recv_ptrs.data_ptr(), self.flag_ptrs.data_ptr(), self.state_ptr
        a.ar_recv_bytes, a.ar_cnt_base, a.pub_ctas = self.recv_half_bytes, self.cnt_base, pub_ctas
        if residual is not None:
            a.residual, a.ldr = residual.data_ptr(), residual.stride(0)
        a.out, a.ldo = out.data_ptr(), out.stride(0)
        if norm_w is not None:
            a.norm_w, a.norm_out, a.ldn = norm_w.data_ptr(), norm_out.data_ptr(), norm_out.stride(0)
            a.eps, a.norm_mode = eps, norm_mode
        a.status = (status if status is not None else self.status).data_ptr()
        a.dtype = 0 if out.dtype == torch.float16 else 1
        return a

    def device_barrier(self) -> None:
        """Bounded device-side barrier over the peer flags (set-up and tests)."""
        N.check(N.lib().rf_peer_barrier(C.c_void_p(self.flag_ptrs.data_ptr()), self.FLAG_COUNT - self.BARRIER_FLAGS,
                                        C.c_void_p(self.state_ptr), self.tp.world, self.tp.rank,
                                        C.c_void_p(self.status.data_ptr()),
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream)), "rf_peer_barrier")

    def argmax_merge(self, vals: torch.Tensor, ids: torch.Tensor, rows: int) -> None:
        """In place: ``ids[:rows]`` becomes the global greedy pick over all ranks' vocab shards."""
        N.check(N.lib().rf_tp_argmax_merge(C.c_void_p(self.aux_ptrs.data_ptr()), C.c_void_p(self.flag_ptrs.data_ptr()),
                                           self.FLAG_COUNT - self.BARRIER_FLAGS + 16, C.c_void_p(self.state_ptr),
                                           self.tp.world, self.tp.rank, rows, self.AUX_ROWS,
                                           C.c_void_p(vals.data_ptr()), C.c_void_p(ids.data_ptr()),
                                           C.c_void_p(self.status.data_ptr()),
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream)), "rf_tp_argmax_merge")

    def close(self) -> None:
        lib = N.lib()
        torch.cuda.synchronize()
        self.tp.barrier()
        for q in self._opened:
            lib.rf_ipc_close(C.c_void_p(q))
        self._opened = []
        if self.local:
            lib.rf_comm_free(C.c_void_p(self.local))
            self.local = 0
