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
