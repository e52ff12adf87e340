"""Build recipe for the native library (the counterpart of the reference's Makefile:150-220,
which runs one nvcc command per kernel).  One shared object, ``libmkernel_b200.so``, is built
in-tree next to this file from the sources under ``csrc/`` for ``sm_100a`` only.

    python -m mkernel_b200.build            # build if sources are newer than the library
    python -m mkernel_b200.build --force
    python -m mkernel_b200.build --shims    # mkernel_b200/shims/lib<name>.so: import shims the
                                            # reference's own load_module.py can load
    python -m mkernel_b200.build --diag     # libmkernel_b200_diag.so: timing diagnostics compiled
                                            # in (-DMKB_DIAG); select it with MKERNEL_B200_LIB
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
DIAG_LIB = PKG / "libmkernel_b200_diag.so"
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


def build_shims(out_dir: Path | str | None = None) -> list[Path]:
    """Compile one import shim per operator module name (csrc/loader_shim.c) into
    ``out_dir/lib<name>.so`` -- the files the reference's unmodified python/load_module.py looks
    for under its ``build/`` directory.  Needs gcc and the CPython headers, not nvcc."""
    import sysconfig

    from .load_module import names
    out = Path(out_dir) if out_dir else PKG / "shims"
    out.mkdir(parents=True, exist_ok=True)
    cc = os.environ.get("CC") or shutil.which("gcc") or shutil.which("cc")
    if not cc:
        raise RuntimeError("no C compiler found for the import shims")
    built = []
    for name in names():
        so = out / f"lib{name}.so"
        cmd = [cc, "-shared", "-fPIC", "-O2", f"-I{sysconfig.get_paths()['include']}",
               f"-DMK_KERNEL={name}", str(CSRC / "loader_shim.c"), "-o", str(so)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"shim build failed:\n{' '.join(cmd)}\n{proc.stderr}")
        built.append(so)
    return built


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def is_stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime_ns for p in list(CSRC.iterdir()) + [PKG.parent / "include" / "mkernel_b200.h"])
    return newest > LIB.stat().st_mtime_ns


def build(force: bool = False, verbose: bool = False, diag: bool = False) -> Path:
    """Compile the library; returns its path.  Raises RuntimeError with the compiler output on
    failure.  diag=True builds the separate diagnostics library (always rebuilt)."""
    lib = DIAG_LIB if diag else LIB
    if not diag and not force and not is_stale():
        return lib
    tmp = lib.with_suffix(f".so.tmp.{os.getpid()}")
    flags = NVCC_FLAGS + (["-DMKB_DIAG"] if diag else [])
    cmd = [_nvcc(), *flags, "-o", str(tmp), *map(str, sources())]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)
    if not diag:
        (PKG / "build_ptxas.log").write_text(proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    return lib


if __name__ == "__main__":
    if "--shims" in sys.argv:
        for p in build_shims():
            print(p)
        sys.exit(0)
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, diag="--diag" in sys.argv)
    print(path)
