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


def _compile(out: Path, extra, verbose: bool) -> Path:
    cmd = [_nvcc(), *NVCC_FLAGS, *extra]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    out.parent.mkdir(parents=True, exist_ok=True)
    cmd += ["-o", str(out), *map(str, SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        print(proc.stderr)
    if proc.returncode:
        raise RuntimeError("nvcc failed:\n" + proc.stderr)
    return out


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    return _compile(LIB, [], verbose)


# The test build: the same library plus the measured alternatives (other tile shapes, two-sweep
# forward, tile-resident backward, chain walkers, vectorised three-phase kernels), selected per
# call through environment variables. Only the GPU tests load it; it lives under tests/.
VARIANTS_LIB = PKG.parent / "tests" / "_variants" / "libfields_read_variants.so"


def build_variants(force: bool = False, verbose: bool = False) -> Path:
    newest = max(p.stat().st_mtime for p in SOURCES + HEADERS)
    if not force and VARIANTS_LIB.exists() and VARIANTS_LIB.stat().st_mtime >= newest:
        return VARIANTS_LIB
    return _compile(VARIANTS_LIB, ["-DFIELDS_ALL_VARIANTS"], verbose)


if __name__ == "__main__":
    import sys
    print(build_library(force=True, verbose="-v" in sys.argv))
