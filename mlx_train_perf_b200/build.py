"""Build recipe of the CUDA shared library (`csrc/` -> `libb200tp.so`, in-tree).

`python -m mlx_train_perf_b200.build` cross-compiles every kernel for sm_100a with nvcc; no
GPU is needed.  The library keeps no link-time dependency on libcuda (the one driver entry
point it needs is resolved at run time), only on the CUDA runtime, which is linked
statically so the .so is self-contained.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
LIB = PKG / "libb200tp.so"

SOURCES = [
    "common.cu",
    "linear_ce_tc.cu",
    "linear_ce_simt.cu",
    "capi_ce.cu",
    "linear_ce_static.cu",
    "flash_simt.cu",
    "flash_tc.cu",
    "capi_attn.cu",
    "selftest.cu",
    "prestep.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]
# The tensor-core kernels use explicit ex2.approx and never rely on libm accuracy; the CUDA-core
# kernels are the fp32-exact path and are compiled without fast-math.
FAST_MATH_SOURCES = {"linear_ce_tc.cu", "flash_tc.cu"}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _digest(path: Path) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    for dep in sorted(list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "b200tp.h"]):
        h.update(dep.read_bytes())
    h.update(" ".join(_flags(path.name)).encode())
    return h.hexdigest()


def _flags(src: str) -> list:
    return NVCC_FLAGS + (["--use_fast_math"] if src in FAST_MATH_SOURCES else [])


def _compile(src: str, verbose: bool) -> Path:
    path = CSRC / src
    obj = OBJ / (path.stem + ".o")
    stamp = OBJ / (path.stem + ".sha")
    dig = _digest(path)
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj
    cmd = [_nvcc(), *_flags(src), "-c", str(path), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = OBJ / (path.stem + ".ptxas.txt")
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stdout.write(f"[build] {src} ok\n")
    stamp.write_text(dig)
    return obj


def build(verbose: bool = True, force: bool = False) -> Path:
    """Compile all sources (in parallel) and link `libb200tp.so` next to the package."""
    OBJ.mkdir(parents=True, exist_ok=True)
    if force:
        for f in OBJ.glob("*.sha"):
            f.unlink()
    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), SOURCES))
    newest = max(o.stat().st_mtime for o in objs)
    if LIB.exists() and LIB.stat().st_mtime >= newest and not force:
        return LIB
    cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static",
           "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stdout.write(f"[build] linked {LIB}\n")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv)
