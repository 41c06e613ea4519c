"""Build librf_b200.so (sm_100a only) in-tree with nvcc.

Usage:  python -m rhinoforge_b200.csrc.build [--force] [--verbose]

Every ``.cu`` / ``.cpp`` under ``csrc/`` becomes one object file under
``csrc/build/`` (cached by a hash of the source, the headers and the flags);
the objects are linked into ``rhinoforge_b200/_native/librf_b200.so``.  The
library has no link-time dependency on libcuda or libtorch, so it also loads on
a machine without a GPU (host-only entry points and planners work there).
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
BUILD = CSRC / "build"
OUT_DIR = PKG / "_native"
LIB = OUT_DIR / "librf_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
          "--expt-relaxed-constexpr", "-Xptxas", "-v", "-diag-suppress", "177,550"]


def nvcc() -> str:
    exe = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; set NVCC or add CUDA to PATH")
    return exe


def sources() -> list[Path]:
    out = []
    for sub in ("common", "kernels", "runtime", "models"):
        d = CSRC / sub
        out += sorted(d.glob("*.cu")) + sorted(d.glob("*.cpp"))
    return out


def headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))):
        if BUILD in p.parents:
            continue
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def compile_one(src: Path, hdig: str, force: bool, verbose: bool, debug: bool) -> tuple[Path, str]:
    flags = ARCH_FLAGS + COMMON + (["-DRF_DEBUG_BOUNDS=1"] if debug else [])
    key = hashlib.sha256(src.read_bytes() + hdig.encode() + " ".join(flags).encode()).hexdigest()[:16]
    obj = BUILD / f"{src.parent.name}_{src.stem}.o"
    stamp = obj.with_suffix(".hash")
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj, ""
    cmd = [nvcc(), *flags, "-I", str(CSRC), "-x", "cu", "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = r.stdout + r.stderr
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{log}")
    stamp.write_text(key)
    (obj.with_suffix(".ptxas.log")).write_text(log)
    return obj, log if verbose else ""


def build(force: bool = False, verbose: bool = False, debug: bool = False, jobs: int | None = None) -> Path:
    BUILD.mkdir(exist_ok=True)
    OUT_DIR.mkdir(exist_ok=True)
    hdig = headers_digest()
    srcs = sources()
    objs: list[Path] = []
    changed = force or not LIB.exists()
    with cf.ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 4)) as ex:
        futs = {ex.submit(compile_one, s, hdig, force, verbose, debug): s for s in srcs}
        for f in cf.as_completed(futs):
            obj, log = f.result()
            objs.append(obj)
            if log:
                print(log)
    newest = max(o.stat().st_mtime for o in objs)
    if changed or not LIB.exists() or LIB.stat().st_mtime < newest:
        tmp = LIB.with_suffix(".so.tmp")
        cmd = [nvcc(), *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, sorted(objs)), "-lcudart_static",
               "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        os.replace(tmp, LIB)
    return LIB


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas -v output")
    ap.add_argument("--debug", action="store_true", help="compile in-kernel bounds checks")
    ap.add_argument("-j", "--jobs", type=int, default=None)
    a = ap.parse_args(argv)
    lib = build(a.force, a.verbose, a.debug, a.jobs)
    print(lib)
    return 0


if __name__ == "__main__":
    sys.exit(main())
