"""ctypes front end of ``field_oracle.c`` (test infrastructure only).

``build()`` compiles the C file with gcc into ``oracle/_build/`` (git-ignored
``.so``); the wrappers take and return numpy arrays with the reference's
layouts: ``raw [B,L,3C]``, ``read [B,L,4C]``, ``grad_read [B,L,4C]``,
``grad_raw [B,L,3C]``, states ``[B,2C]``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path
from typing import Optional, Tuple

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "field_oracle.c"
_OUT = _HERE / "_build" / "libfield_oracle.so"
_LIB: Optional[ctypes.CDLL] = None


def build(force: bool = False) -> Path:
    """Compile the C oracle if the shared object is missing or stale."""
    if not force and _OUT.exists() and _OUT.stat().st_mtime >= _SRC.stat().st_mtime:
        return _OUT
    _OUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-o", str(_OUT), str(_SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return _OUT


def _lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = build()
        lib = ctypes.CDLL(str(path))
        p = ctypes.c_void_p
        i = ctypes.c_int
        lib.field_oracle_forward.argtypes = [p, p, p, p, p, p, p, i, i, i]
        lib.field_oracle_forward.restype = i
        lib.field_oracle_backward.argtypes = [p] * 12 + [i, i, i]
        lib.field_oracle_backward.restype = i
        lib.field_oracle_span_summary.argtypes = [p] * 5 + [i, i, i]
        lib.field_oracle_span_summary.restype = i
        _LIB = lib
    return _LIB


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x), dtype=np.float32)


def _f64_or_none(x) -> Optional[np.ndarray]:
    return None if x is None else np.ascontiguousarray(np.asarray(x), dtype=np.float64)


def _ptr(x: Optional[np.ndarray]):
    return None if x is None else x.ctypes.data_as(ctypes.c_void_p)


def forward(raw, tr, ti, gamma, state_in=None) -> Tuple[np.ndarray, np.ndarray]:
    """Returns ``(read [B,L,4C] float64, state_out [B,2C] float64)``."""
    raw, tr, ti, gamma = _f32(raw), _f32(tr), _f32(ti), _f32(gamma)
    B, L, C3 = raw.shape
    C = tr.size
    if C3 != 3 * C:
        raise ValueError((raw.shape, tr.shape))
    state_in = _f64_or_none(state_in)
    read = np.zeros((B, L, 4 * C), dtype=np.float64)
    state_out = np.zeros((B, 2 * C), dtype=np.float64)
    rc = _lib().field_oracle_forward(_ptr(raw), _ptr(tr), _ptr(ti), _ptr(gamma),
                                     _ptr(state_in), _ptr(read), _ptr(state_out), B, L, C)
    if rc:
        raise RuntimeError(f"field_oracle_forward failed with code {rc}")
    return read, state_out


def backward(raw, tr, ti, gamma, grad_read, state_in=None, grad_state_out=None):
    """Returns ``(grad_raw, grad_tr, grad_ti, grad_gamma, grad_state_in)`` in float64."""
    raw, tr, ti, gamma = _f32(raw), _f32(tr), _f32(ti), _f32(gamma)
    grad_read = _f32(grad_read)
    B, L, C3 = raw.shape
    C = tr.size
    if C3 != 3 * C or grad_read.shape != (B, L, 4 * C):
        raise ValueError((raw.shape, grad_read.shape, tr.shape))
    state_in = _f64_or_none(state_in)
    grad_state_out = _f64_or_none(grad_state_out)
    grad_raw = np.zeros((B, L, 3 * C), dtype=np.float64)
    gtr = np.zeros(C, dtype=np.float64)
    gti = np.zeros(C, dtype=np.float64)
    ggm = np.zeros(C, dtype=np.float64)
    gsi = np.zeros((B, 2 * C), dtype=np.float64)
    rc = _lib().field_oracle_backward(_ptr(raw), _ptr(tr), _ptr(ti), _ptr(gamma),
                                      _ptr(state_in), _ptr(grad_read), _ptr(grad_state_out),
                                      _ptr(grad_raw), _ptr(gtr), _ptr(gti), _ptr(ggm),
                                      _ptr(gsi), B, L, C)
    if rc:
        raise RuntimeError(f"field_oracle_backward failed with code {rc}")
    return grad_raw, gtr, gti, ggm, gsi


def span_summary(raw, tr, ti, gamma) -> np.ndarray:
    """Affine summary ``[B,4,C]`` (Re A | Im A | Re Bv | Im Bv) of the whole span."""
    raw, tr, ti, gamma = _f32(raw), _f32(tr), _f32(ti), _f32(gamma)
    B, L, C3 = raw.shape
    C = tr.size
    out = np.zeros((B, 4, C), dtype=np.float64)
    rc = _lib().field_oracle_span_summary(_ptr(raw), _ptr(tr), _ptr(ti), _ptr(gamma),
                                          _ptr(out), B, L, C)
    if rc:
        raise RuntimeError(f"field_oracle_span_summary failed with code {rc}")
    return out


def num_threads() -> int:
    """Threads the OpenMP loops will use (for reporting next to timings)."""
    env = os.environ.get("OMP_NUM_THREADS")
    return int(env) if env else (os.cpu_count() or 1)


if __name__ == "__main__":
    print(build(force=True))
