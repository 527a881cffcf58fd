"""Loads ``libfields_read.so`` and declares the C ABI of ``include/fields_read.h``.

There is no fallback: if the CUDA library has not been built, loading raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libfields_read.so"

_P = ctypes.c_void_p
_I = ctypes.c_int
_SZ = ctypes.c_size_t
_LL = ctypes.c_longlong

# name -> (restype, argtypes); every symbol include/fields_read.h declares
SYMBOLS = {
    "fields_status_string": (ctypes.c_char_p, [_I]),
    "fields_read_version": (_I, []),
    "fields_last_cuda_error": (ctypes.c_char_p, []),
    "fields_read_workspace_bytes": (_SZ, [_I, _I, _I, _I]),
    "fields_read_forward": (_I, [_P] * 8 + [_SZ, _I, _I, _I, _P]),
    "fields_read_backward": (_I, [_P] * 14 + [_SZ, _I, _I, _I, _P]),
    "fields_read_state_rows": (_I, [_I]),
    "fields_read_backward_from_states": (_I, [_P] * 14 + [_SZ, _I, _I, _I, _P]),
    "fields_read_forward_bf16": (_I, [_P] * 8 + [_SZ, _I, _I, _I, _P]),
    "fields_read_forward_bf16_tensor": (_I, [_P] * 8 + [_I, _I, _I, _P]),
    "fields_read_forward_bf16_stats": (_I, [_P] * 9 + [_SZ, _I, _I, _I, _P]),
    "fields_read_backward_bf16": (_I, [_P] * 14 + [_SZ, _I, _I, _I, _P]),
    "fields_read_device_status": (_I, [_P, _P]),
    "fields_read_selftest_wait": (_I, [_P, _SZ, ctypes.c_uint, _P]),
    "fields_read_step": (_I, [_P] * 6 + [_I, _I, _P]),
    "fields_read_step_bf16": (_I, [_P] * 6 + [_I, _I, _P]),
    "fields_scan_workspace_bytes": (_SZ, [_I, _I, _I]),
    "fields_scan_forward": (_I, [_P, _LL, _LL, _I] + [_P] * 5 + [_SZ, _I, _I, _I, _P]),
    "fields_scan_backward": (_I, [_P, _LL, _LL, _I] + [_P] * 8 + [_SZ, _I, _I, _I, _P]),
    "fields_read_span_summary": (_I, [_P] * 6 + [_SZ, _I, _I, _I, _P]),
    "fields_read_fold_summaries": (_I, [_P, _P, _P, _I, _I, _I, _I, _P]),
    "fields_read_span_summary_backward": (_I, [_P] * 6 + [_SZ, _I, _I, _I, _P]),
    "fields_read_fold_summaries_backward": (_I, [_P, _P, _P, _I, _I, _I, _I, _P]),
    "fields_read_mailbox_bytes": (_SZ, [_I, _I, _I]),
    "fields_read_span_summary_put": (_I, [_P] * 6 + [_I, _I, ctypes.c_uint, _P, _SZ, _I, _I, _I, _P]),
    "fields_read_forward_sharded": (_I, [_P] * 10 + [_I, _I, ctypes.c_uint, ctypes.c_uint,
                                              _I, _I, _I, _P]),
    "fields_read_fold_mailbox": (_I, [_P, _P, _P, _P, _I, _I, ctypes.c_uint, ctypes.c_uint, _I, _I, _P]),
    "fields_read_sum_over_ranks": (_I, [_P, _P, _I, _P, _P, _I, _I, ctypes.c_uint, ctypes.c_uint,
                                       _I, _I, _P]),
    "fields_read_span_summary_backward_put": (_I, [_P] * 6 + [_I, _I, ctypes.c_uint, _P, _SZ, _I, _I, _I, _P]),
    "fields_read_fold_mailbox_backward": (_I, [_P, _P, _P, _P, _I, _I, ctypes.c_uint, ctypes.c_uint, _I, _I, _P]),
    "fields_read_norm_grad_combine": (_I, [_P, _P, _P, _P, ctypes.c_longlong, _I, _P]),
    "fields_mixer_epilogue_bias_rows": (_SZ, [ctypes.c_longlong]),
    "fields_mixer_epilogue_forward": (_I, [_P] * 7 + [ctypes.c_float, _I, ctypes.c_longlong, _I, _P]),
    "fields_mixer_epilogue_backward": (_I, [_P] * 11 + [ctypes.c_float, _I, ctypes.c_longlong, _I, _P]),
    "fields_read_static_scratch_bytes": (_SZ, []),
    "fields_read_forward_noalloc": (_I, [_P] * 7 + [_I, _I, _I, _P]),
}

_lib = None


class FieldsLibraryError(RuntimeError):
    """The CUDA library is missing or a call into it returned a non-zero status."""


def open_library(path: Path) -> ctypes.CDLL:
    """Opens a build of the library and declares every symbol of the C ABI on it."""
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise FieldsLibraryError(
            f"{LIB_PATH.name} has not been built; run `python -m fields_lm_b200.build` "
            "(needs nvcc). There is no CPU fallback for the Field kernels.")
    _lib = open_library(LIB_PATH)
    return _lib


def check(status: int, what: str) -> None:
    if status:
        lib = load()
        text = lib.fields_status_string(status).decode()
        if status == 3:
            text += ": " + lib.fields_last_cuda_error().decode()
        raise FieldsLibraryError(f"{what}: {text} (status {status})")
