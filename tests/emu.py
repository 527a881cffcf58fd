"""Host emulation of the CUDA library for the CPU test-suite (test infrastructure).

Compiles ``fields_lm_b200/csrc/fields_read.cu`` with g++ and FIELDS_HOST_EMU:
every kernel launch becomes a loop over (block, phase, thread) on host memory.
The exported C ABI is the same, so the tests drive it exactly as they drive the
CUDA library, with numpy arrays in place of device buffers. The package never
loads this build.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "fields_lm_b200" / "csrc" / "fields_read.cu"
OUT = ROOT / "tests" / "_emu" / "libfields_read_emu.so"
_LIB = None

P = ctypes.c_void_p
I = ctypes.c_int
SZ = ctypes.c_size_t


def build() -> Path:
    deps = list((ROOT / "fields_lm_b200" / "csrc").glob("*")) + [ROOT / "include" / "fields_read.h"]
    if OUT.exists() and OUT.stat().st_mtime >= max(d.stat().st_mtime for d in deps):
        return OUT
    OUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = ["g++", "-x", "c++", "-std=c++17", "-O2", "-fPIC", "-shared", "-DFIELDS_HOST_EMU", "-DFIELDS_ALL_VARIANTS",
           "-Wall", "-Wno-unknown-pragmas", "-Wno-maybe-uninitialized", "-o", str(OUT), str(SRC)]
    subprocess.run(cmd, check=True)
    return OUT


def declare(lib: ctypes.CDLL) -> ctypes.CDLL:
    """ctypes signatures of include/fields_read.h (shared with the real library's tests)."""
    lib.fields_status_string.argtypes = [I]
    lib.fields_status_string.restype = ctypes.c_char_p
    lib.fields_read_version.restype = I
    lib.fields_read_workspace_bytes.argtypes = [I, I, I, I]
    lib.fields_read_workspace_bytes.restype = SZ
    lib.fields_read_forward.argtypes = [P] * 8 + [SZ, I, I, I, P]
    lib.fields_read_forward.restype = I
    lib.fields_read_backward.argtypes = [P] * 14 + [SZ, I, I, I, P]
    lib.fields_read_backward.restype = I
    lib.fields_read_state_rows.argtypes = [I]
    lib.fields_read_state_rows.restype = I
    lib.fields_read_backward_from_states.argtypes = [P] * 14 + [SZ, I, I, I, P]
    lib.fields_read_backward_from_states.restype = I
    lib.fields_read_forward_bf16.argtypes = [P] * 8 + [SZ, I, I, I, P]
    lib.fields_read_forward_bf16.restype = I
    lib.fields_read_forward_bf16_stats.argtypes = [P] * 9 + [SZ, I, I, I, P]
    lib.fields_read_forward_bf16_stats.restype = I
    lib.fields_read_backward_bf16.argtypes = [P] * 14 + [SZ, I, I, I, P]
    lib.fields_read_backward_bf16.restype = I
    lib.fields_read_span_summary.argtypes = [P] * 6 + [SZ, I, I, I, P]
    lib.fields_read_span_summary.restype = I
    lib.fields_read_fold_summaries.argtypes = [P, P, P, I, I, I, I, P]
    lib.fields_read_fold_summaries.restype = I
    lib.fields_read_span_summary_backward.argtypes = [P] * 6 + [SZ, I, I, I, P]
    lib.fields_read_span_summary_backward.restype = I
    lib.fields_read_fold_summaries_backward.argtypes = [P, P, P, I, I, I, I, P]
    lib.fields_read_fold_summaries_backward.restype = I
    lib.fields_read_step.argtypes = [P] * 6 + [I, I, P]
    lib.fields_read_step.restype = I
    lib.fields_read_step_bf16.argtypes = [P] * 6 + [I, I, P]
    lib.fields_read_step_bf16.restype = I
    lib.fields_read_selftest_wait.argtypes = [P, SZ, ctypes.c_uint, P]
    lib.fields_read_selftest_wait.restype = I
    lib.fields_read_mailbox_bytes.argtypes = [I, I, I]
    lib.fields_read_mailbox_bytes.restype = SZ
    lib.fields_read_span_summary_put.argtypes = [P] * 6 + [I, I, ctypes.c_uint, P, SZ, I, I, I, P]
    lib.fields_read_span_summary_put.restype = I
    lib.fields_read_fold_mailbox.argtypes = [P, P, P, P, I, I, ctypes.c_uint, ctypes.c_uint, I, I, P]
    lib.fields_read_fold_mailbox.restype = I
    lib.fields_read_span_summary_backward_put.argtypes = [P] * 6 + [I, I, ctypes.c_uint, P, SZ, I, I, I, P]
    lib.fields_read_span_summary_backward_put.restype = I
    lib.fields_read_fold_mailbox_backward.argtypes = [P, P, P, P, I, I, ctypes.c_uint, ctypes.c_uint, I, I, P]
    lib.fields_read_fold_mailbox_backward.restype = I
    lib.fields_read_forward_sharded.argtypes = [P] * 10 + [I, I, ctypes.c_uint, ctypes.c_uint,
                                                   I, I, I, P]
    lib.fields_read_forward_sharded.restype = I
    lib.fields_read_sum_over_ranks.argtypes = [P, P, I, P, P, I, I, ctypes.c_uint, ctypes.c_uint, I, I, P]
    lib.fields_read_sum_over_ranks.restype = I
    lib.fields_read_device_status.argtypes = [P, P]
    lib.fields_read_device_status.restype = I
    LL = ctypes.c_longlong
    lib.fields_scan_workspace_bytes.argtypes = [I, I, I]
    lib.fields_scan_workspace_bytes.restype = SZ
    lib.fields_scan_forward.argtypes = [P, LL, LL, I] + [P] * 5 + [SZ, I, I, I, P]
    lib.fields_scan_forward.restype = I
    lib.fields_scan_backward.argtypes = [P, LL, LL, I] + [P] * 8 + [SZ, I, I, I, P]
    lib.fields_scan_backward.restype = I
    return lib


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = declare(ctypes.CDLL(str(build())))
    return _LIB


def _aligned(nbytes: int, align: int = 256) -> np.ndarray:
    buf = np.zeros(nbytes + align, dtype=np.uint8)
    off = (-buf.ctypes.data) % align
    return buf[off:off + nbytes]


def _f32(x, align=256):
    x = np.asarray(x, dtype=np.float32)
    out = _aligned(max(x.nbytes, 4), align).view(np.float32)[:x.size].reshape(x.shape)
    out[...] = x
    return out


def _ptr(a):
    return None if a is None else a.ctypes.data_as(P)


def forward(raw, tr, ti, gamma, state_in=None, want_state=True, misalign=False,
            return_workspace=False):
    """Runs the emulated forward. ``misalign`` offsets raw by 4 bytes to force the scalar path."""
    B, L, C3 = raw.shape
    C = tr.size
    if misalign:
        store = _f32(np.concatenate([[0.0], np.asarray(raw, np.float32).ravel()]))
        raw_a = store[1:].reshape(raw.shape)
    else:
        raw_a = _f32(raw)
    tr_a, ti_a, gm_a = _f32(tr), _f32(ti), _f32(gamma)
    sin_a = None if state_in is None else _f32(state_in)
    read = _f32(np.full((B, L, 4 * C), np.nan))
    sout = _f32(np.full((B, 2 * C), np.nan)) if want_state else None
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 0)
    ws = _aligned(max(nbytes, 256))
    ws[...] = 0xFF  # poison: nothing may rely on a zeroed workspace
    rc = lib().fields_read_forward(_ptr(raw_a), _ptr(tr_a), _ptr(ti_a), _ptr(gm_a), _ptr(sin_a),
                                   _ptr(read), _ptr(sout), _ptr(ws), nbytes, B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    if return_workspace:
        return read, sout, ws
    return read, sout


def backward(raw, tr, ti, gamma, read, grad_read, state_in=None, grad_state_out=None):
    B, L, C3 = raw.shape
    C = tr.size
    a = [_f32(x) for x in (raw, tr, ti, gamma)]
    sin_a = None if state_in is None else _f32(state_in)
    gso_a = None if grad_state_out is None else _f32(grad_state_out)
    read_a, gr_a = _f32(read), _f32(grad_read)
    g_raw = _f32(np.full((B, L, 3 * C), np.nan))
    g_tr, g_ti, g_gm = (_f32(np.full(C, np.nan)) for _ in range(3))
    g_sin = _f32(np.full((B, 2 * C), np.nan))
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 1)
    ws = _aligned(max(nbytes, 256))
    ws[...] = 0xFF
    rc = lib().fields_read_backward(_ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(a[3]), _ptr(sin_a),
                                    _ptr(read_a), _ptr(gr_a), _ptr(gso_a), _ptr(g_raw), _ptr(g_tr),
                                    _ptr(g_ti), _ptr(g_gm), _ptr(g_sin), _ptr(ws), nbytes,
                                    B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return g_raw, g_tr, g_ti, g_gm, g_sin


def backward_from_states(raw, tr, ti, gamma, read, grad_read, state_in=None, grad_state_out=None):
    """Backward that is given only every eighth state row of `read` (taken from it here)."""
    B, L, C3 = raw.shape
    C = tr.size
    rows = lib().fields_read_state_rows(L)
    states = _f32(np.ascontiguousarray(np.asarray(read)[:, 7::8, :2 * C][:, :rows])) if rows else None
    a = [_f32(x) for x in (raw, tr, ti, gamma)]
    sin_a = None if state_in is None else _f32(state_in)
    gso_a = None if grad_state_out is None else _f32(grad_state_out)
    gr_a = _f32(grad_read)
    g_raw = _f32(np.full((B, L, 3 * C), np.nan))
    g_tr, g_ti, g_gm = (_f32(np.full(C, np.nan)) for _ in range(3))
    g_sin = _f32(np.full((B, 2 * C), np.nan))
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 1)
    ws = _aligned(max(nbytes, 256))
    ws[...] = 0xFF
    rc = lib().fields_read_backward_from_states(
        _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(a[3]), _ptr(sin_a), _ptr(states), _ptr(gr_a),
        _ptr(gso_a), _ptr(g_raw), _ptr(g_tr), _ptr(g_ti), _ptr(g_gm), _ptr(g_sin), _ptr(ws), nbytes,
        B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return g_raw, g_tr, g_ti, g_gm, g_sin


def span_summary(raw, tr, ti, gamma):
    B, L, C3 = raw.shape
    C = tr.size
    a = [_f32(x) for x in (raw, tr, ti, gamma)]
    out = _f32(np.full((B, 4, C), np.nan))
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 0)
    ws = _aligned(max(nbytes, 256))
    ws[...] = 0xFF
    rc = lib().fields_read_span_summary(_ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(a[3]), _ptr(out),
                                        _ptr(ws), nbytes, B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out


def fold_summaries(summaries, rank, state0=None):
    P_, B, four, C = summaries.shape
    s = _f32(summaries)
    s0 = None if state0 is None else _f32(state0)
    out = _f32(np.full((B, 2 * C), np.nan))
    rc = lib().fields_read_fold_summaries(_ptr(s), _ptr(s0), _ptr(out), rank, P_, B, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out


def span_summary_backward(raw, tr, ti, grad_read):
    B, L, C3 = raw.shape
    C = tr.size
    a = [_f32(x) for x in (raw, tr, ti, grad_read)]
    out = _f32(np.full((B, 4, C), np.nan))
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 1)
    ws = _aligned(max(nbytes, 256))
    ws[...] = 0xFF
    rc = lib().fields_read_span_summary_backward(_ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(a[3]),
                                                 _ptr(out), _ptr(ws), nbytes, B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out


def fold_summaries_backward(summaries, rank, carry_end=None):
    P_, B, four, C = summaries.shape
    s = _f32(summaries)
    c0 = None if carry_end is None else _f32(carry_end)
    out = _f32(np.full((B, 2 * C), np.nan))
    rc = lib().fields_read_fold_summaries_backward(_ptr(s), _ptr(c0), _ptr(out), rank, P_, B, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out


def step(raw_row, tr, ti, gamma, state, bf16=False):
    """One decode step; returns (read_row, new_state). With bf16, raw/read are uint16 bit patterns."""
    B, C3 = raw_row.shape
    C = tr.size
    a = [_f32(x) for x in (tr, ti, gamma)]
    st = _f32(state)
    if bf16:
        store = _aligned(B * C3 * 2).view(np.uint16).reshape(B, C3)
        store[...] = raw_row
        out = _aligned(B * 4 * C * 2).view(np.uint16).reshape(B, 4 * C)
        rc = lib().fields_read_step_bf16(_ptr(store), _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(st),
                                         _ptr(out), B, C, None)
    else:
        r = _f32(raw_row)
        out = _f32(np.full((B, 4 * C), np.nan))
        rc = lib().fields_read_step(_ptr(r), _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(st),
                                    _ptr(out), B, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out, st


def _u16(x, fill=None):
    """Aligned uint16 copy of a bf16 bit pattern array (or an output buffer of that shape)."""
    x = np.asarray(x, dtype=np.uint16)
    out = _aligned(max(x.nbytes, 8)).view(np.uint16)[:x.size].reshape(x.shape)
    out[...] = x if fill is None else fill
    return out


def forward_bf16(raw_bits, tr, ti, gamma):
    B, L, C3 = raw_bits.shape
    C = tr.size
    r = _u16(raw_bits)
    a = [_f32(x) for x in (tr, ti, gamma)]
    read = _u16(np.zeros((B, L, 4 * C), np.uint16), fill=0x7fc0)
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 0)
    ws = _aligned(max(nbytes, 256))
    rc = lib().fields_read_forward_bf16(_ptr(r), _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), None, _ptr(read),
                                        None, _ptr(ws), nbytes, B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return read


def forward_bf16_stats(raw_bits, tr, ti, gamma):
    """Returns (read bits, sumsq [B, L, G])."""
    B, L, C3 = raw_bits.shape
    C = tr.size
    G = (C + 127) // 128
    r = _u16(raw_bits)
    a = [_f32(x) for x in (tr, ti, gamma)]
    read = _u16(np.zeros((B, L, 4 * C), np.uint16), fill=0x7fc0)
    sumsq = _f32(np.full((B, L, G), np.nan))
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 0)
    ws = _aligned(max(nbytes, 256))
    rc = lib().fields_read_forward_bf16_stats(_ptr(r), _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), None,
                                              _ptr(read), _ptr(sumsq), None, _ptr(ws), nbytes,
                                              B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return read, sumsq


def backward_bf16(raw_bits, tr, ti, gamma, read_bits, grad_bits):
    B, L, C3 = raw_bits.shape
    C = tr.size
    r, rd, g = _u16(raw_bits), _u16(read_bits), _u16(grad_bits)
    a = [_f32(x) for x in (tr, ti, gamma)]
    g_raw = _u16(np.zeros((B, L, 3 * C), np.uint16), fill=0x7fc0)
    g_tr, g_ti, g_gm = (_f32(np.full(C, np.nan)) for _ in range(3))
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 1)
    ws = _aligned(max(nbytes, 256))
    rc = lib().fields_read_backward_bf16(_ptr(r), _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), None, _ptr(rd),
                                         _ptr(g), None, _ptr(g_raw), _ptr(g_tr), _ptr(g_ti), _ptr(g_gm),
                                         None, _ptr(ws), nbytes, B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return g_raw, g_tr, g_ti, g_gm


def make_mailboxes(world, B, C):
    """One zeroed mailbox per emulated rank (all in host memory, so every 'peer' can write them)."""
    n = lib().fields_read_mailbox_bytes(world, B, C)
    return [_aligned(n) for _ in range(world)]


def span_summary_put(raw, tr, ti, gamma, mailboxes, rank, epoch):
    B, L, C3 = raw.shape
    C = tr.size
    a = [_f32(x) for x in (raw, tr, ti, gamma)]
    ptrs = (ctypes.c_void_p * len(mailboxes))(*[m.ctypes.data for m in mailboxes])
    out = _f32(np.full((B, 4, C), np.nan))
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 0)
    ws = _aligned(max(nbytes, 256))
    rc = lib().fields_read_span_summary_put(_ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(a[3]), ptrs,
                                            _ptr(out), rank, len(mailboxes), epoch, _ptr(ws), nbytes,
                                            B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out


def span_summary_backward_put(raw, tr, ti, grad_read, mailboxes, rank, epoch):
    B, L, C3 = raw.shape
    C = tr.size
    a = [_f32(x) for x in (raw, tr, ti, grad_read)]
    ptrs = (ctypes.c_void_p * len(mailboxes))(*[m.ctypes.data for m in mailboxes])
    out = _f32(np.full((B, 4, C), np.nan))
    nbytes = lib().fields_read_workspace_bytes(B, L, C, 1)
    ws = _aligned(max(nbytes, 256))
    rc = lib().fields_read_span_summary_backward_put(_ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(a[3]),
                                                     ptrs, _ptr(out), rank, len(mailboxes), epoch,
                                                     _ptr(ws), nbytes, B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out


def fold_mailbox_backward(mailbox, rank, world, epoch, B, C, carry_end=None):
    c0 = None if carry_end is None else _f32(carry_end)
    out = _f32(np.full((B, 2 * C), np.nan))
    err = np.zeros(1, dtype=np.uint32)
    rc = lib().fields_read_fold_mailbox_backward(_ptr(mailbox), _ptr(c0), _ptr(out), _ptr(err), rank,
                                                 world, epoch, 0, B, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out, int(err[0])


def fold_mailbox(mailbox, rank, world, epoch, B, C, state0=None):
    s0 = None if state0 is None else _f32(state0)
    out = _f32(np.full((B, 2 * C), np.nan))
    err = np.zeros(1, dtype=np.uint32)
    rc = lib().fields_read_fold_mailbox(_ptr(mailbox), _ptr(s0), _ptr(out), _ptr(err), rank, world,
                                        epoch, 0, B, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return out, int(err[0])


class ShardedForward:
    """One emulated rank of ``fields_read_forward_sharded``: buffers that live across the two
    halves of the launch, which a test runs apart (all ranks' first sweeps, then all waits)."""

    def __init__(self, raw, tr, ti, gamma, mailboxes, rank, state0=None):
        self.B, self.L, _ = raw.shape
        self.C = tr.size
        self.a = [_f32(x) for x in (raw, tr, ti, gamma)]
        self.s0 = None if state0 is None else _f32(state0)
        self.read = _f32(np.full((self.B, self.L, 4 * self.C), np.nan))
        self.state = _f32(np.full((self.B, 2 * self.C), np.nan))
        self.summary = _f32(np.full((self.B, 4, self.C), np.nan))
        self.err = np.zeros(1, dtype=np.uint32)
        self.ptrs = (ctypes.c_void_p * len(mailboxes))(*[m.ctypes.data for m in mailboxes])
        self.world, self.rank = len(mailboxes), rank

    def run(self, stages, epoch):
        lib().fields_emu_span_stages(stages)
        try:
            rc = lib().fields_read_forward_sharded(
                _ptr(self.a[0]), _ptr(self.a[1]), _ptr(self.a[2]), _ptr(self.a[3]), _ptr(self.s0),
                _ptr(self.read), _ptr(self.state), _ptr(self.summary), self.ptrs, _ptr(self.err),
                self.rank, self.world, epoch, 0, self.B, self.L, self.C, None)
        finally:
            lib().fields_emu_span_stages(3)
        if rc:
            raise RuntimeError(lib().fields_status_string(rc).decode())
        return self


def forward_bf16_tensor(raw_bits, tr, ti, gamma, state_in=None):
    """The tensor-core experiment's forward with the contraction emulated by a plain loop over the
    same shared-memory operand layouts. Returns (read bits, state_out, error word)."""
    B, L, C3 = raw_bits.shape
    C = tr.size
    raw_a = _u16(raw_bits)
    a = [_f32(x) for x in (tr, ti, gamma)]
    s_in = None if state_in is None else _f32(state_in)
    read = _u16(np.zeros((B, L, 4 * C), np.uint16), fill=0x7FC0)
    state = _f32(np.full((B, 2 * C), np.nan))
    err = np.zeros(1, dtype=np.uint32)
    fn = lib().fields_read_forward_bf16_tensor
    fn.argtypes = [P] * 8 + [I, I, I, P]
    fn.restype = I
    rc = fn(_ptr(raw_a), _ptr(a[0]), _ptr(a[1]), _ptr(a[2]), _ptr(s_in), _ptr(read), _ptr(state),
            _ptr(err), B, L, C, None)
    if rc:
        raise RuntimeError(lib().fields_status_string(rc).decode())
    return read, state, int(err[0])


def _scan_layout(a, B, L, C):
    """(buffer, batch stride, step stride, channel stride) of a dense [B, L, C] or per-token
    [B, L] decay, as fields_scan_forward takes it."""
    a = _f32(a)
    return (a, L, 1, 0) if a.ndim == 2 else (a, L * C, C, 1)


def scan_forward(a, b, state_in=None, want_state=True):
    """Emulated fields_scan_forward; ``a`` is [B, L, C] or one decay per token [B, L]."""
    b = _f32(b)
    B, L, C = b.shape
    a, ab, at, ac = _scan_layout(a, B, L, C)
    sin = None if state_in is None else _f32(state_in)
    states = _f32(np.full((B, L, C), np.nan))
    sout = _f32(np.full((B, C), np.nan)) if want_state else None
    nbytes = lib().fields_scan_workspace_bytes(B, L, C)
    ws = _aligned(max(nbytes, 16))
    rc = lib().fields_scan_forward(_ptr(a), ab, at, ac, _ptr(b), _ptr(sin), _ptr(states),
                                   _ptr(sout), _ptr(ws), nbytes, B, L, C, None)
    assert rc == 0, rc
    return states, sout


def scan_backward(a, states, grad_states, state_in=None, grad_state_out=None, want_state_grad=False):
    """Emulated fields_scan_backward. Returns (grad_a dense, grad_b, grad_state_in or None)."""
    states, g = _f32(states), _f32(grad_states)
    B, L, C = states.shape
    a, ab, at, ac = _scan_layout(a, B, L, C)
    sin = None if state_in is None else _f32(state_in)
    gso = None if grad_state_out is None else _f32(grad_state_out)
    ga, gb = _f32(np.full((B, L, C), np.nan)), _f32(np.full((B, L, C), np.nan))
    gsi = _f32(np.full((B, C), np.nan)) if want_state_grad else None
    nbytes = lib().fields_scan_workspace_bytes(B, L, C)
    ws = _aligned(max(nbytes, 16))
    rc = lib().fields_scan_backward(_ptr(a), ab, at, ac, _ptr(states), _ptr(sin), _ptr(g),
                                    _ptr(gso), _ptr(ga), _ptr(gb), _ptr(gsi), _ptr(ws), nbytes,
                                    B, L, C, None)
    assert rc == 0, rc
    return ga, gb, gsi


def sum_over_ranks(values_by_rank, mailboxes, epoch, B, C, absent=()):
    """Emulated fields_read_sum_over_ranks for all ranks of a job: first every present rank's
    stores, then every present rank's wait-and-add. Returns ([sum per rank], [error word per rank])."""
    world = len(mailboxes)
    ptrs = (ctypes.c_void_p * world)(*[m.ctypes.data for m in mailboxes])
    vals = [_f32(v) for v in values_by_rank]
    outs = [_f32(np.full(v.shape, np.nan)) for v in vals]
    errs = [np.zeros(1, dtype=np.uint32) for _ in range(world)]
    try:
        for stages in (1, 2):
            lib().fields_emu_span_stages(stages)
            for r in range(world):
                if r in absent:
                    continue
                rc = lib().fields_read_sum_over_ranks(_ptr(vals[r]), _ptr(outs[r]), vals[r].size, ptrs,
                                                      _ptr(errs[r]), r, world, epoch, 0, B, C, None)
                assert rc == 0, rc
    finally:
        lib().fields_emu_span_stages(3)
    return outs, [int(e[0]) for e in errs]
