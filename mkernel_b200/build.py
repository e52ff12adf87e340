"""Build recipe for the native library (the counterpart of the reference's Makefile:150-220,
which runs one nvcc command per kernel).  One shared object, ``libmkernel_b200.so``, is built
in-tree next to this file from the sources under ``csrc/`` for ``sm_100a`` only.

    python -m mkernel_b200.build            # build if sources are newer than the library
    python -m mkernel_b200.build --force
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libmkernel_b200.so"
SOURCES = ["ops.cu", "transport.cpp"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add the CUDA toolkit to PATH")


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def is_stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime_ns for p in list(CSRC.iterdir()) + [PKG.parent / "include" / "mkernel_b200.h"])
    return newest > LIB.stat().st_mtime_ns


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library; returns its path.  Raises RuntimeError with the compiler output on
    failure."""
    if not force and not is_stale():
        return LIB
    tmp = LIB.with_suffix(f".so.tmp.{os.getpid()}")
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(tmp), *map(str, sources())]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB)
    (PKG / "build_ptxas.log").write_text(proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
