"""Failure detection without a GPU fault: failures are made on the host (a rank that exits or raises,
an undersized buffer, an error code from the native layer) and must surface as an error, never a hang."""
import ctypes as C
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _launch(scenario: str, tmp_path: Path, world: int = 2, timeout: int = 120):
    env = os.environ.copy()
    env.update({"MASTER_ADDR": "127.0.0.1", "CUDA_VISIBLE_DEVICES": ""})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29641", str(ROOT / "tests" / "_fault_worker.py"), scenario, str(tmp_path / "r")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    reports = {int(p.suffixes[0][5:]): json.loads(p.read_text()) for p in tmp_path.glob("r.rank*.json")}
    return r, reports


def test_rank_that_exits_between_steps_is_reported_before_the_next_launch(tmp_path):
    r, reports = _launch("rank_exits_between_steps", tmp_path)
    rep = reports[0]
    assert rep["step0"] == "ok"
    # rank 1 published step 1 and left; rank 0 passes step 1 and is told at step 2 -- on the host, within the limit
    assert rep.get("step1") == "ok"
    assert rep["step2"].startswith("error:") and "rank(s) [1]" in rep["step2"]


def test_rank_that_stalls_on_the_host_is_detected_within_the_timeout(tmp_path):
    r, reports = _launch("rank_stalls_on_host", tmp_path)
    assert reports[0]["result"] == "detected" and "rank(s) [1]" in reports[0]["message"]
    assert reports[0]["seconds"] < 3.0
    assert reports[1]["result"] == "woke up"


def _lib():
    from rhinoforge_b200 import _native as N
    if not N.available():
        pytest.skip("native library not built")
    return N, N.lib()


def test_undersized_allreduce_buffer_is_rejected_on_the_host():
    """The fused all-reduce needs room for every rank's partial; a short buffer is an argument error
    raised before any launch (no GPU is touched: this runs on a CPU-only machine)."""
    N, lib = _lib()
    g = N.RfGemm()
    g.x, g.w, g.out = 0x1000, 0x2000, 0x3000
    g.ldx = g.ldw = 4096
    g.ldo = 4096
    g.M, g.N, g.K = 64, 4096, 4096
    g.ar_world, g.ar_rank = 8, 0
    g.ar_recv, g.ar_flags, g.ar_state = 0x4000, 0x5000, 0x6000
    g.ar_recv_bytes, g.ar_flag_count = 1024, 1 << 20           # far too small for 8 x 64 x 4096 fp32
    g.force_swap = -1
    rc = lib.rf_gemm(C.byref(g), None)
    assert rc != 0
    msg = lib.rf_last_error().decode()
    assert "receive buffer too small" in msg


def test_stack_rejects_an_unbound_or_undersized_arena():
    N, lib = _lib()
    sc = N.RfStackConfig()
    sc.layers, sc.hidden, sc.Hq, sc.Hkv, sc.hd, sc.inter = 1, 256, 4, 2, 64, 512
    sc.max_tokens, sc.max_seqs, sc.true_hd, sc.tp_world = 64, 2, 64, 1
    h = C.c_int64(lib.rf_stack_create(C.byref(sc)))
    assert h.value >= 0
    need = lib.rf_stack_arena_bytes(h)
    assert need > 0
    rc = lib.rf_stack_bind_arena(h, C.c_void_p(0x10000), C.c_uint64(need // 2))
    assert rc != 0 and b"arena" in lib.rf_last_error()
    f = N.RfStackForward()
    f.hidden, f.tokens, f.num_seqs = 0x20000, 8, 1
    rc = lib.rf_stack_forward(h, C.byref(f), None)
    assert rc != 0 and b"arena is not bound" in lib.rf_last_error()
    lib.rf_stack_destroy(h)


def test_native_errors_become_python_exceptions_with_the_message():
    N, lib = _lib()
    from rhinoforge_b200.runtime.errors import RPUBackendError
    g = N.RfGemm()                                  # all-null arguments
    rc = lib.rf_gemm(C.byref(g), None)
    with pytest.raises(RPUBackendError, match="GEMM needs x, w and out"):
        N.check(rc, "rf_gemm")


def test_allreduce_protocol_model_sums_in_rank_order_and_survives_a_rank_one_call_ahead():
    """Host model of the in-kernel protocol: both variants give every rank the same bits, over several back-to-back
    calls (slot alternation), with one rank deliberately slow."""
    import time
    import numpy as np
    from rhinoforge_b200.parallel.protocol_sim import SimWorld, run_ranks
    rng = np.random.default_rng(0)
    for two_shot in (False, True):
        W = 4
        world = SimWorld(W, rows=6, cols=16, tile_cols=4, wait_s=2.0)
        for call in range(3):
            parts = [rng.standard_normal((6, 16)).astype(np.float32) for _ in range(W)]
            resid = rng.standard_normal((6, 16)).astype(np.float32)

            def one(rank):
                if rank == 2:
                    time.sleep(0.05)                      # a slow rank: the others wait on its flags
                return world.all_reduce(rank, parts[rank], resid, two_shot=two_shot)
            outs = run_ranks(world, one)
            if two_shot:
                want = sum(p.astype(np.float16).astype(np.float32) for p in parts) + resid
                tol = 2e-2
            else:
                want = ((parts[0] + parts[1]) + parts[2]) + parts[3] + resid
                tol = 1e-6
            for o in outs:
                assert o is not None and np.allclose(o, want, atol=tol)
                assert np.array_equal(o, outs[0]), "every rank must hold the same bits"
        assert all(m.status == 0 and m.call == 3 for m in world.mem)


def test_allreduce_protocol_model_times_out_instead_of_hanging_when_a_flag_is_withheld():
    """A flag write that never arrives (dropped on the host) ends the waiters' call with the peer-timeout status
    within the wait bound; the other tiles still complete and the next call works again."""
    import time
    import numpy as np
    from rhinoforge_b200.parallel.protocol_sim import STATUS_PEER_TIMEOUT, SimWorld, run_ranks
    W = 2
    world = SimWorld(W, rows=2, cols=8, tile_cols=4, wait_s=0.2)
    world.allow_flag = lambda kind, src, dst, tile: not (kind == 0 and src == 1 and dst == 0 and tile == 1)
    parts = [np.full((2, 8), float(r + 1), np.float32) for r in range(W)]
    t0 = time.monotonic()
    outs = run_ranks(world, lambda r: world.all_reduce(r, parts[r], None, two_shot=False))
    assert time.monotonic() - t0 < 2.0
    assert outs[0] is None and world.mem[0].status == STATUS_PEER_TIMEOUT and world.mem[0].status_detail == 1
    assert outs[1] is not None and np.allclose(outs[1], 3.0)          # rank 1 got every flag
    world.allow_flag = lambda *a: True
    for m in world.mem:
        m.status = 0
    outs = run_ranks(world, lambda r: world.all_reduce(r, parts[r], None, two_shot=True))
    assert all(o is not None and np.allclose(o, 3.0) for o in outs)
