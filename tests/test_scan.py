"""The real-valued scan (the softpatch mixer's call of ``hierarchical_scan``) on the CPU:
the oracle against fixtures made by the reference's own function, and the kernels of
``field_scan.cuh`` through the host emulation against the oracle."""
import numpy as np
import pytest

import emu
from conftest import GOLDEN, rel_err
from oracle import scan_oracle

PIN_TOL = 2e-6


@pytest.fixture(scope="module")
def golden_scan():
    return np.load(GOLDEN / "scan_small.npz")


def _case(g, name):
    return {k: g[f"{name}/{k}"] for k in ("a", "b", "grad_states", "states", "grad_a", "grad_b")}


def _expanded(a, b):
    return a[..., None] if a.ndim == 2 else a


@pytest.mark.parametrize("idx", range(6))
def test_oracle_matches_the_reference_function(golden_scan, idx):
    c = _case(golden_scan, str(golden_scan["cases"][idx]))
    a = _expanded(c["a"], c["b"])
    states, last = scan_oracle.forward(a, c["b"])
    assert rel_err(states, c["states"]) < PIN_TOL
    np.testing.assert_array_equal(last, states[:, -1])
    grad_a, grad_b, _ = scan_oracle.backward(a, c["b"], c["grad_states"])
    if c["a"].ndim == 2:                       # autograd sums over the expanded channels
        grad_a = grad_a.sum(axis=2)
    assert rel_err(grad_b, c["grad_b"]) < PIN_TOL
    assert rel_err(grad_a, c["grad_a"]) < 5e-6


@pytest.mark.parametrize("idx", range(6))
def test_emulated_kernels_match_the_fixtures(golden_scan, idx):
    c = _case(golden_scan, str(golden_scan["cases"][idx]))
    states, last = emu.scan_forward(c["a"], c["b"])
    assert rel_err(states, c["states"]) < 1e-5
    np.testing.assert_array_equal(last, states[:, -1])
    grad_a, grad_b, _ = emu.scan_backward(c["a"], states, c["grad_states"])
    if c["a"].ndim == 2:
        grad_a = grad_a.astype(np.float64).sum(axis=2)
    assert rel_err(grad_b, c["grad_b"]) < 1e-5
    assert rel_err(grad_a, c["grad_a"]) < 1e-5


@pytest.mark.parametrize("B,L,C,per_token", [(2, 257, 64, True), (1, 16, 32, False),
                                              (3, 15, 33, False), (2, 1000, 7, True),
                                              (1, 17, 1, False)])
def test_emulated_kernels_with_state_in_and_out(B, L, C, per_token):
    rng = np.random.default_rng(L * 31 + C)
    a = rng.uniform(0.01, 0.99, (B, L) if per_token else (B, L, C)).astype(np.float32)
    b = rng.standard_normal((B, L, C)).astype(np.float32)
    sin = rng.standard_normal((B, C)).astype(np.float32)
    g = rng.standard_normal((B, L, C)).astype(np.float32)
    gso = rng.standard_normal((B, C)).astype(np.float32)
    wide = a[..., None] if per_token else a
    want, want_last = scan_oracle.forward(wide, b, sin)
    states, last = emu.scan_forward(a, b, sin)
    assert rel_err(states, want) < 1e-5 and rel_err(last, want_last) < 1e-5
    wa, wb, wsi = scan_oracle.backward(wide, b, g, sin, gso)
    ga, gb, gsi = emu.scan_backward(a, states, g, sin, gso, want_state_grad=True)
    assert rel_err(ga, wa) < 1e-5 and rel_err(gb, wb) < 1e-5 and rel_err(gsi, wsi) < 1e-5


def test_spans_chain_through_the_state():
    """Two calls over the halves of a sequence, the second from the first's end state, equal
    one call over the whole (what a sequence-sharded or incremental caller relies on)."""
    rng = np.random.default_rng(5)
    a = rng.uniform(0.2, 0.99, (2, 90, 12)).astype(np.float32)
    b = rng.standard_normal((2, 90, 12)).astype(np.float32)
    whole, last = emu.scan_forward(a, b)
    first, mid = emu.scan_forward(a[:, :41], b[:, :41])
    second, end = emu.scan_forward(a[:, 41:], b[:, 41:], mid)
    assert rel_err(np.concatenate([first, second], axis=1), whole) < 2e-6
    assert rel_err(end, last) < 2e-6


def test_empty_and_argument_errors():
    lib = emu.lib()
    assert lib.fields_scan_workspace_bytes(0, 5, 5) == 0
    a = emu._f32(np.ones((1, 4, 4)))
    out = emu._f32(np.zeros((1, 4, 4)))
    ws = emu._aligned(max(lib.fields_scan_workspace_bytes(1, 4, 4), 16))
    args = (emu._ptr(a), 16, 4, 1, emu._ptr(a), None, emu._ptr(out), None)
    assert lib.fields_scan_forward(*args, emu._ptr(ws), ws.nbytes, 1, 4, 4, None) == 0
    assert lib.fields_scan_forward(*args, emu._ptr(ws), 8, 1, 4, 4, None) == 2        # workspace
    assert lib.fields_scan_forward(*args, None, ws.nbytes, 1, 4, 4, None) == 2
    bad = (emu._ptr(a), 16, 4, 2, emu._ptr(a), None, emu._ptr(out), None)             # channel stride
    assert lib.fields_scan_forward(*bad, emu._ptr(ws), ws.nbytes, 1, 4, 4, None) == 1
    assert lib.fields_scan_forward(*args, emu._ptr(ws), ws.nbytes, 1, 4, 0, None) == 1
    assert lib.fields_scan_forward(*args, emu._ptr(ws), ws.nbytes, 0, 4, 4, None) == 0  # empty batch
    # no steps: the state passes through
    sin = emu._f32(np.arange(4, dtype=np.float32).reshape(1, 4))
    sout = emu._f32(np.zeros((1, 4)))
    rc = lib.fields_scan_forward(None, 0, 0, 1, None, emu._ptr(sin), None, emu._ptr(sout), None, 0,
                                 1, 0, 4, None)
    assert rc == 0
    np.testing.assert_array_equal(sout, sin)
