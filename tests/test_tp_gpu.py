"""Tensor parallelism on real GPUs: the fused GEMM + all-reduce kernel and the sharded engine."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _run(world: int, tmp_path: Path) -> None:
    env = os.environ.copy()
    env.update({"NCCL_NVLS_ENABLE": "0", "RF_TP_REPORT": str(tmp_path / "tp"), "MASTER_ADDR": "127.0.0.1"})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), str(ROOT / "tests" / "_tp_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    reports = "\n".join(p.read_text() for p in sorted(tmp_path.glob("tp.rank*.json")))
    assert r.returncode == 0, f"{r.stdout[-3000:]}\n{r.stderr[-3000:]}\n{reports[-6000:]}"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_allreduce_and_sharded_engine(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, tmp_path)
