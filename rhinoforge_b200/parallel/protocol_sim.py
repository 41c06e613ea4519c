"""Host model of the in-kernel all-reduce protocol (threads stand in for GPUs, numpy arrays for peer memory).

The fused GEMM epilogue (``csrc/kernels/gemm_tc.cu``) talks to its peers through three pieces of symmetric memory per
rank - a double-buffered receive area, a flag array and a call counter - with these rules:

* one-shot (up to 256 rows): every rank stores its fp32 partial of a tile into slot ``call & 1`` of EVERY rank's receive
  area, publishes flag ``(tile, source)`` = ``call + 1`` on every rank with release semantics, waits (bounded) until its
  own flags of all sources reach ``call + 1``, sums the partials in rank order and adds the residual;
* two-shot (more rows): the partial (16-bit) goes to the tile's owner ``tile % world`` only; the owner waits for all
  sources, reduces, writes the finished tile into every rank's result region and publishes a second flag; every rank
  waits for that flag and copies the tile out;
* a wait that runs out sets a status word and returns - the kernel never spins forever;
* flags carry the call number, so nothing is ever reset, and consecutive calls alternate slots, so a rank that is one
  call ahead cannot overwrite data a slower rank still reads.

This module replays those rules on the host so that the protocol itself - ordering, slot reuse, time-outs - is testable
without a GPU and without faulting one: a test can withhold a flag, delay a rank or run many calls back to back.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import numpy as np

STATUS_OK, STATUS_PEER_TIMEOUT = 0, 5


@dataclass
class RankMemory:
    """What one rank exposes to its peers."""
    recv: np.ndarray            # [2 slots, world + 1 regions, rows, cols] fp32 (region `world` = two-shot results)
    flags: np.ndarray           # [2 kinds, tiles, world] int64: kind 0 "partial landed", kind 1 "result landed"
    call: int = 0
    status: int = STATUS_OK
    status_detail: int = -1
    lock: threading.Lock = field(default_factory=threading.Lock)


class SimWorld:
    def __init__(self, world: int, rows: int, cols: int, tile_cols: int = 4, wait_s: float = 0.5):
        assert cols % tile_cols == 0
        self.world, self.rows, self.cols, self.tile_cols, self.wait_s = world, rows, cols, tile_cols, wait_s
        self.tiles = cols // tile_cols
        self.mem = [RankMemory(np.zeros((2, world + 1, rows, cols), np.float32), np.zeros((2, self.tiles, world), np.int64))
                    for _ in range(world)]
        # hooks for fault injection: return False to drop that flag write
        self.allow_flag: Callable[[int, int, int, int], bool] = lambda kind, src, dst, tile: True

    # -- primitives with the kernel's semantics --------------------------------------------------------------
    def _release_flag(self, kind: int, src: int, dst: int, tile: int, value: int) -> None:
        if self.allow_flag(kind, src, dst, tile):
            m = self.mem[dst]
            with m.lock:                      # the lock models release/acquire ordering of the flag itself
                m.flags[kind, tile, src] = value

    def _wait_flag(self, rank: int, kind: int, tile: int, src: int, want: int) -> bool:
        m = self.mem[rank]
        deadline = time.monotonic() + self.wait_s
        while time.monotonic() < deadline:
            with m.lock:
                if m.flags[kind, tile, src] >= want:
                    return True
            time.sleep(0.0005)
        m.status, m.status_detail = STATUS_PEER_TIMEOUT, src
        return False

    # -- one call of one rank ----------------------------------------------------------------------------------
    def all_reduce(self, rank: int, partial: np.ndarray, residual: Optional[np.ndarray], *, two_shot: bool) -> Optional[np.ndarray]:
        """Run one fused all-reduce as ``rank``; returns the reduced ``[rows, cols]`` array or None after a time-out."""
        W, me = self.world, self.mem[rank]
        call = me.call
        slot, want = call & 1, call + 1
        out = np.zeros((self.rows, self.cols), np.float32)
        ok = True
        for t in range(self.tiles):
            c0, c1 = t * self.tile_cols, (t + 1) * self.tile_cols
            if not two_shot:
                for dst in range(W):
                    self.mem[dst].recv[slot, rank, :, c0:c1] = partial[:, c0:c1]
                for dst in range(W):
                    self._release_flag(0, rank, dst, t, want)
                if not all(self._wait_flag(rank, 0, t, src, want) for src in range(W)):
                    ok = False
                    continue
                acc = np.zeros((self.rows, c1 - c0), np.float32)
                for src in range(W):                       # rank order: every rank computes the same bits
                    acc += me.recv[slot, src, :, c0:c1]
                out[:, c0:c1] = acc + (residual[:, c0:c1] if residual is not None else 0.0)
            else:
                owner = t % W
                self.mem[owner].recv[slot, rank, :, c0:c1] = partial[:, c0:c1].astype(np.float16)
                self._release_flag(0, rank, owner, t, want)
                if rank == owner:
                    if all(self._wait_flag(rank, 0, t, src, want) for src in range(W)):
                        acc = np.zeros((self.rows, c1 - c0), np.float32)
                        for src in range(W):
                            acc += me.recv[slot, src, :, c0:c1]
                        acc += residual[:, c0:c1] if residual is not None else 0.0
                        for dst in range(W):
                            self.mem[dst].recv[slot, W, :, c0:c1] = acc.astype(np.float16)
                        for dst in range(W):
                            self._release_flag(1, rank, dst, t, want)
                    else:
                        ok = False
                if not self._wait_flag(rank, 1, t, owner, want):
                    ok = False
                    continue
                out[:, c0:c1] = me.recv[slot, W, :, c0:c1]
        me.call = call + 1                                  # the last CTA advances the call counter, time-out or not
        return out if ok else None


def run_ranks(world: SimWorld, fn: Callable[[int], object]) -> List[object]:
    """Run ``fn(rank)`` on one thread per rank and return the results in rank order."""
    res: List[object] = [None] * world.world

    def body(r: int) -> None:
        res[r] = fn(r)
    threads = [threading.Thread(target=body, args=(r,)) for r in range(world.world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return res


__all__ = ["SimWorld", "run_ranks", "STATUS_OK", "STATUS_PEER_TIMEOUT"]
