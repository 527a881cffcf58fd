"""Pins the CPU oracles to fixtures produced by the reference's own code.

The fixtures hold outputs of the reference's ``reference_field_read`` and of
autograd through it (see tests/golden/make_golden.py). Both restatements - the
sequential double-precision C oracle and the complex64 PyTorch port - must
reproduce them. The reference computes in fp32, so the bound is a few fp32
roundings, far inside the 1e-5 parity tolerance.
"""
import numpy as np
import pytest
import torch

from conftest import rel_err
from oracle import field_oracle, torch_port

PIN_TOL = 2e-6


def _case(g, name):
    return {k: g[f"{name}/{k}"] for k in
            ("raw", "tr", "ti", "gamma", "grad_read", "read", "grad_raw",
             "grad_tr", "grad_ti", "grad_gamma")}


def test_fixture_cases_present(golden_small):
    assert len(golden_small["cases"]) >= 6


@pytest.mark.parametrize("idx", range(7))
def test_c_oracle_matches_reference_small(golden_small, idx):
    c = _case(golden_small, str(golden_small["cases"][idx]))
    read, state = field_oracle.forward(c["raw"], c["tr"], c["ti"], c["gamma"])
    assert rel_err(read, c["read"]) < PIN_TOL
    C = c["tr"].size
    np.testing.assert_array_equal(state, read[:, -1, :2 * C])
    g_raw, g_tr, g_ti, g_gm, _ = field_oracle.backward(
        c["raw"], c["tr"], c["ti"], c["gamma"], c["grad_read"])
    assert rel_err(g_raw, c["grad_raw"]) < PIN_TOL
    assert rel_err(g_tr, c["grad_tr"]) < 5e-6
    assert rel_err(g_ti, c["grad_ti"]) < 5e-6
    assert rel_err(g_gm, c["grad_gamma"]) < 5e-6


@pytest.mark.parametrize("idx", range(7))
def test_torch_port_matches_reference_small(golden_small, idx):
    c = _case(golden_small, str(golden_small["cases"][idx]))
    t = {k: torch.from_numpy(v.copy()) for k, v in c.items()}
    raw = t["raw"].requires_grad_(True)
    tr, ti, gm = (t[k].requires_grad_(True) for k in ("tr", "ti", "gamma"))
    read = torch_port.field_read(raw, tr, ti, gm, 32)
    read.backward(t["grad_read"])
    assert rel_err(read.detach().numpy(), c["read"]) < PIN_TOL
    assert rel_err(raw.grad.numpy(), c["grad_raw"]) < PIN_TOL
    assert rel_err(tr.grad.numpy(), c["grad_tr"]) < 5e-6
    assert rel_err(ti.grad.numpy(), c["grad_ti"]) < 5e-6
    assert rel_err(gm.grad.numpy(), c["grad_gamma"]) < 5e-6


def test_c_oracle_matches_reference_config1(golden_config1):
    g = golden_config1
    steps = g["steps"]
    read, _ = field_oracle.forward(g["raw"], g["tr"], g["ti"], g["gamma"])
    assert rel_err(read[:, steps], g["read_steps"]) < PIN_TOL
    g_raw, g_tr, g_ti, g_gm, _ = field_oracle.backward(
        g["raw"], g["tr"], g["ti"], g["gamma"], g["grad_read"].astype(np.float32))
    assert rel_err(g_raw[:, steps], g["grad_raw_steps"]) < PIN_TOL
    assert rel_err(g_tr, g["grad_tr"]) < 5e-6
    assert rel_err(g_ti, g["grad_ti"]) < 5e-6
    assert rel_err(g_gm, g["grad_gamma"]) < 5e-6


def test_state_in_chains_spans():
    """Running two spans with the carried state equals one pass (causality)."""
    rng = np.random.default_rng(5)
    B, L, C = 2, 50, 12
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    radius = rng.uniform(0.5, 0.999, C).astype(np.float32)
    theta = rng.uniform(-3, 3, C).astype(np.float32)
    tr, ti = radius * np.cos(theta), radius * np.sin(theta)
    gm = np.sqrt(1 - radius ** 2).astype(np.float32)
    full, end = field_oracle.forward(raw, tr, ti, gm)
    a, mid = field_oracle.forward(raw[:, :21], tr, ti, gm)
    b, end2 = field_oracle.forward(raw[:, 21:], tr, ti, gm, state_in=mid)
    np.testing.assert_allclose(np.concatenate([a, b], 1), full, rtol=0, atol=1e-14)
    np.testing.assert_allclose(end2, end, rtol=0, atol=1e-14)
    # the span summary applied to the incoming state gives the outgoing state
    s = field_oracle.span_summary(raw[:, 21:], tr, ti, gm)
    A = s[:, 0] + 1j * s[:, 1]
    Bv = s[:, 2] + 1j * s[:, 3]
    m = mid[:, :C] + 1j * mid[:, C:]
    e = end[:, :C] + 1j * end[:, C:]
    np.testing.assert_allclose(A * m + Bv, e, rtol=0, atol=1e-13)


def test_backward_matches_finite_differences():
    rng = np.random.default_rng(11)
    B, L, C = 1, 9, 3
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    radius = rng.uniform(0.6, 0.95, C).astype(np.float32)
    theta = rng.uniform(-2, 2, C).astype(np.float32)
    tr, ti = radius * np.cos(theta), radius * np.sin(theta)
    gm = np.sqrt(1 - radius ** 2).astype(np.float32)
    w = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    s_in = rng.standard_normal((B, 2 * C))
    w_end = rng.standard_normal((B, 2 * C))

    def loss(raw_, s_in_):
        r, e = field_oracle.forward(raw_, tr, ti, gm, state_in=s_in_)
        return float((r * w).sum() + (e * w_end).sum())

    g_raw, _, _, _, g_sin = field_oracle.backward(raw, tr, ti, gm, w, state_in=s_in,
                                                  grad_state_out=w_end)
    eps = 1e-2  # raw is float32 inside the oracle; a coarse step keeps the difference exact
    for idx in [(0, 0, 0), (0, 4, 5), (0, 8, 8), (0, 3, 7)]:
        p, m = raw.copy(), raw.copy()
        p[idx] += eps
        m[idx] -= eps
        fd = (loss(p, s_in) - loss(m, s_in)) / (float(p[idx]) - float(m[idx]))
        assert abs(fd - g_raw[idx]) < 2e-3 * max(1.0, abs(fd))
    for idx in [(0, 0), (0, 4)]:
        p, m = s_in.copy(), s_in.copy()
        p[idx] += 1e-6
        m[idx] -= 1e-6
        fd = (loss(raw, p) - loss(raw, m)) / 2e-6
        assert abs(fd - g_sin[idx]) < 1e-6 * max(1.0, abs(fd))
