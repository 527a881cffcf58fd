"""Builds ``libfields_read.so`` (CUDA, sm_100a) next to this file.

``python -m fields_lm_b200.build`` or :func:`build_library`. nvcc cross-compiles
without a GPU; the shared object stays in-tree (ignored by git).
"""
from __future__ import annotations

import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libfields_read.so"
SOURCES = [CSRC / "fields_read.cu"]
HEADERS = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "fields_read.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-ftz=true",  # denormals flush to zero: far below the parity bound, saves instructions
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def is_stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in SOURCES + HEADERS)
    return LIB.stat().st_mtime < newest


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB), *map(str, SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        print(proc.stderr)
    if proc.returncode:
        raise RuntimeError("nvcc failed:\n" + proc.stderr)
    return LIB


if __name__ == "__main__":
    import sys
    print(build_library(force=True, verbose="-v" in sys.argv))
