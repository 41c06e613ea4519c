#!/usr/bin/env python3
"""Check that the package imports, the native library loads and a B200 is reachable."""
from __future__ import annotations

import sys
from pathlib import Path


def main() -> int:
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import torch
    import rpu_backend
    from rhinoforge_b200 import _native
    print(f"rpu_backend {rpu_backend.__version__} (torch {torch.__version__})")
    print(f"native library: {'built' if _native.available() else 'missing'} at {_native.LIB_PATH}")
    if not torch.cuda.is_available():
        print("no CUDA device visible: host-only mode (planners, converters and config checks work)")
        return 0
    name = torch.cuda.get_device_name(0)
    cc = torch.cuda.get_device_capability(0)
    print(f"device 0: {name} (sm_{cc[0]}{cc[1]}), torch.rpu.is_available() = {torch.rpu.is_available()}")
    if cc[0] != 10:
        print("warning: the kernels are built for sm_100a only")
        return 1
    from rhinoforge_b200.ops import kernels as K
    x = torch.randn(4, 256, device="cuda").half()
    w = torch.randn(128, 256, device="cuda").half()
    err = (K.gemm(x, w).float() - x.float() @ w.float().t()).abs().max().item()
    print(f"tcgen05 GEMM self-check: max abs error {err:.4f}")
    return 0 if err < 0.1 else 1


if __name__ == "__main__":
    raise SystemExit(main())
