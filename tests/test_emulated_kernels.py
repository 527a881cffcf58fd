"""Runs the CUDA kernels' own source on the host (see tests/emu.py) against the oracle.

This checks, without a GPU, the launch plan, every index computation and every
formula of the shipped kernels. The fp32 parity bound (1e-5 relative) is applied
here too.
"""
import numpy as np
import pytest

import emu
from conftest import BF16_TOL, FP32_TOL, rel_err
from oracle import field_oracle


def _params(C, rng):
    radius = rng.uniform(0.5, 0.99995, C).astype(np.float32)
    theta = rng.uniform(-np.pi, np.pi, C).astype(np.float32)
    return (radius * np.cos(theta)).astype(np.float32), (radius * np.sin(theta)).astype(np.float32), \
        np.sqrt(np.maximum(1 - radius ** 2, 1e-4)).astype(np.float32)


ALGOS = [("three_phase", "0", "forward"), ("single_pass", "0", "forward"),
         ("single_pass", "0", "reverse"), ("single_pass", "1", "forward"),
         ("single_pass", "1", "reverse"), ("single_pass", "2", "forward"),
         ("single_pass", "2", "reverse"), ("single_pass", "3", "forward"),
         ("single_pass", "3", "reverse"),
         ("walk", "0", "forward")]


@pytest.fixture(params=ALGOS, ids=lambda a: "-".join(a))
def algo(request, monkeypatch):
    """Selects the kernel family, the tuning variant of the single-pass kernels (forward and
    backward alike) and the order in which emulated blocks finish."""
    name, variant, order = request.param
    monkeypatch.setenv("FIELDS_READ_ALGO", name)
    monkeypatch.setenv("FIELDS_FWD_VARIANT", variant)
    monkeypatch.setenv("FIELDS_BWD_VARIANT", variant)
    monkeypatch.setenv("FIELDS_EMU_ORDER", order)
    return request.param


SHAPES = [(1, 1, 4), (2, 37, 32), (3, 130, 20), (1, 64, 4), (2, 65, 12), (2, 33, 7),
          (1, 48, 160), (1, 300, 132), (2, 16, 512), (5, 17, 1)]


@pytest.mark.parametrize("B,L,C", SHAPES)
@pytest.mark.parametrize("with_state", [False, True])
def test_forward_backward_against_oracle(B, L, C, with_state, algo):
    rng = np.random.default_rng(B * 1000 + L * 10 + C)
    tr, ti, gm = _params(C, rng)
    raw = (rng.standard_normal((B, L, 3 * C)) * 1.5).astype(np.float32)
    grad_read = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    s_in = rng.standard_normal((B, 2 * C)).astype(np.float32) if with_state else None
    g_out = rng.standard_normal((B, 2 * C)).astype(np.float32) if with_state else None

    ref_read, ref_state = field_oracle.forward(raw, tr, ti, gm, state_in=s_in)
    read, state = emu.forward(raw, tr, ti, gm, state_in=s_in)
    assert rel_err(read, ref_read) < FP32_TOL
    assert rel_err(state, ref_state) < FP32_TOL

    ref = field_oracle.backward(raw, tr, ti, gm, grad_read, state_in=s_in, grad_state_out=g_out)
    got = emu.backward(raw, tr, ti, gm, read, grad_read, state_in=s_in, grad_state_out=g_out)
    names = ("grad_raw", "grad_tr", "grad_ti", "grad_gamma", "grad_state_in")
    for name, a, b in zip(names, got, ref):
        assert rel_err(a, b) < FP32_TOL, name


def test_scalar_path_equals_vector_path():
    rng = np.random.default_rng(3)
    B, L, C = 2, 70, 24
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    a, sa = emu.forward(raw, tr, ti, gm)
    b, sb = emu.forward(raw, tr, ti, gm, misalign=True)
    # the scalar path is the three-phase kernels: same arithmetic, different association
    assert rel_err(a, b) < 1e-6
    assert rel_err(sa, sb) < 1e-6


def test_golden_small_cases(golden_small, algo):
    for name in golden_small["cases"]:
        c = {k: golden_small[f"{name}/{k}"] for k in
             ("raw", "tr", "ti", "gamma", "grad_read", "read", "grad_raw", "grad_tr", "grad_ti",
              "grad_gamma")}
        read, _ = emu.forward(c["raw"], c["tr"], c["ti"], c["gamma"])
        assert rel_err(read, c["read"]) < FP32_TOL, name
        g = emu.backward(c["raw"], c["tr"], c["ti"], c["gamma"], read, c["grad_read"])
        assert rel_err(g[0], c["grad_raw"]) < FP32_TOL, name
        assert rel_err(g[1], c["grad_tr"]) < FP32_TOL, name
        assert rel_err(g[2], c["grad_ti"]) < FP32_TOL, name
        assert rel_err(g[3], c["grad_gamma"]) < FP32_TOL, name


def test_long_sequence_many_chunks(algo):
    """More chunks than carry-scan warps, ragged tail, several channel groups."""
    rng = np.random.default_rng(9)
    B, L, C = 1, 16 * 37 + 5, 136
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    ref, _ = field_oracle.forward(raw, tr, ti, gm)
    read, _ = emu.forward(raw, tr, ti, gm)
    assert rel_err(read, ref) < FP32_TOL


def test_single_pass_status_word_is_clear(monkeypatch):
    monkeypatch.setenv("FIELDS_READ_ALGO", "single_pass")
    rng = np.random.default_rng(4)
    B, L, C = 2, 200, 132
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    read, _, ws = emu.forward(raw, tr, ti, gm, return_workspace=True)
    assert emu.lib().fields_read_device_status(ws.ctypes.data_as(emu.P), None) == 0
    assert not np.isnan(read).any()


def test_empty_inputs():
    C = 8
    tr = ti = gm = np.ones(C, np.float32)
    read, state = emu.forward(np.zeros((2, 0, 3 * C), np.float32), tr, ti, gm,
                              state_in=np.full((2, 2 * C), 3.0, np.float32))
    assert read.shape == (2, 0, 4 * C)
    np.testing.assert_array_equal(state, 3.0)
    g = emu.backward(np.zeros((2, 0, 3 * C), np.float32), tr, ti, gm,
                     np.zeros((2, 0, 4 * C), np.float32), np.zeros((2, 0, 4 * C), np.float32),
                     grad_state_out=np.full((2, 2 * C), 2.0, np.float32))
    np.testing.assert_array_equal(g[1], 0.0)
    np.testing.assert_array_equal(g[4], 2.0)


def test_bad_arguments_return_status():
    L = emu.lib()
    assert L.fields_read_forward(None, None, None, None, None, None, None, None, 0, 1, 4, 4, None) == 1
    assert L.fields_read_forward(None, None, None, None, None, None, None, None, 0, 1, 4, 0, None) == 1
    assert L.fields_read_workspace_bytes(0, 5, 4, 0) == 0
    assert L.fields_read_workspace_bytes(2, 100, 512, 1) > L.fields_read_workspace_bytes(2, 100, 512, 0)
    assert b"workspace" in L.fields_status_string(2)


@pytest.mark.parametrize("B,L,C", [(2, 333, 20), (1, 64, 512), (3, 17, 7)])
def test_span_summary_and_fold(B, L, C):
    """Spans summarised separately and folded in order give the state a single pass reaches."""
    rng = np.random.default_rng(L + C)
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    s0 = rng.standard_normal((B, 2 * C)).astype(np.float32)
    assert rel_err(emu.span_summary(raw, tr, ti, gm), field_oracle.span_summary(raw, tr, ti, gm)) < FP32_TOL
    cuts = [0, L // 3, L // 3 + 1, L]
    spans = [raw[:, a:b] for a, b in zip(cuts[:-1], cuts[1:]) if b > a]
    summaries = np.stack([emu.span_summary(x, tr, ti, gm) for x in spans])
    state = s0.astype(np.float64)
    for r, x in enumerate(spans):
        got = emu.fold_summaries(summaries, r, state0=s0)
        assert rel_err(got, state) < FP32_TOL
        _, state = field_oracle.forward(x, tr, ti, gm, state_in=state)
    np.testing.assert_array_equal(emu.fold_summaries(summaries, 0), 0.0)


@pytest.mark.parametrize("B,L,C", [(2, 333, 20), (1, 64, 512), (3, 17, 7)])
def test_backward_over_spans_equals_one_backward_pass(B, L, C):
    """Dual summaries folded in reverse span order give every span the gradient carry a single
    backward pass would hand it; span backward passes then add up to the full one."""
    rng = np.random.default_rng(3 * L + C)
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    grad = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    s0 = rng.standard_normal((B, 2 * C)).astype(np.float32)
    g_end = rng.standard_normal((B, 2 * C)).astype(np.float32)
    want = field_oracle.backward(raw, tr, ti, gm, grad, state_in=s0, grad_state_out=g_end)
    cuts = [0, L // 3, L // 3 + 1, L]
    spans = [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]
    fwd = np.stack([emu.span_summary(raw[:, a:b], tr, ti, gm) for a, b in spans])
    dual = np.stack([emu.span_summary_backward(raw[:, a:b], tr, ti, grad[:, a:b]) for a, b in spans])
    g_raw = np.zeros((B, L, 3 * C), np.float32)
    g_par = [np.zeros(C, np.float64) for _ in range(3)]
    g_in = None
    for r, (a, b) in enumerate(spans):
        state_in = emu.fold_summaries(fwd, r, state0=s0)
        carry = emu.fold_summaries_backward(dual, r, carry_end=g_end)
        read, _ = emu.forward(raw[:, a:b], tr, ti, gm, state_in=state_in)
        out = emu.backward(raw[:, a:b], tr, ti, gm, read, grad[:, a:b], state_in=state_in,
                           grad_state_out=carry)
        g_raw[:, a:b] = out[0]
        for k in range(3):
            g_par[k] += out[1 + k]
        if r == 0:
            g_in = out[4]
    assert rel_err(g_raw, want[0]) < FP32_TOL
    for k in range(3):
        assert rel_err(g_par[k], want[1 + k]) < FP32_TOL
    assert rel_err(g_in, want[4]) < FP32_TOL
    # the last span's carry is the caller's; no carry and no later span gives zero
    np.testing.assert_array_equal(emu.fold_summaries_backward(dual, len(spans) - 1), 0.0)


@pytest.mark.parametrize("B,L,C", [(2, 130, 20), (1, 300, 132), (2, 8, 4), (3, 9, 512), (1, 64, 4)])
@pytest.mark.parametrize("with_state", [False, True])
@pytest.mark.parametrize("order", ["forward", "reverse"])
def test_backward_from_saved_state_rows(monkeypatch, B, L, C, with_state, order):
    """Backward that sees every eighth state only equals the backward that reads all of `read`."""
    monkeypatch.setenv("FIELDS_EMU_ORDER", order)
    rng = np.random.default_rng(B * L + C)
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    grad = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    s0 = rng.standard_normal((B, 2 * C)).astype(np.float32) if with_state else None
    g_end = rng.standard_normal((B, 2 * C)).astype(np.float32) if with_state else None
    read, _ = emu.forward(raw, tr, ti, gm, state_in=s0)
    got = emu.backward_from_states(raw, tr, ti, gm, read, grad, state_in=s0, grad_state_out=g_end)
    want = field_oracle.backward(raw, tr, ti, gm, grad, state_in=s0, grad_state_out=g_end)
    for g, w in zip(got[:4], want[:4]):
        assert rel_err(g, w) < FP32_TOL
    if with_state:
        assert rel_err(got[4], want[4]) < FP32_TOL


def test_backward_from_saved_state_rows_refuses_what_it_cannot_do():
    rng = np.random.default_rng(0)
    tr, ti, gm = _params(7, rng)
    raw = rng.standard_normal((1, 20, 21)).astype(np.float32)
    grad = rng.standard_normal((1, 20, 28)).astype(np.float32)
    read, _ = emu.forward(raw, tr, ti, gm)
    with pytest.raises(RuntimeError):  # channel count not a multiple of four
        emu.backward_from_states(raw, tr, ti, gm, read, grad)


def test_saturated_gates_and_slowest_decay(algo):
    """Saturating inputs, exact zeros, vacancy pinned at both ends, every channel at the largest
    radius: forward and backward of every kernel family and variant against the oracle."""
    rng = np.random.default_rng(99)
    B, L, C = 2, 300, 20
    radius = np.full(C, 0.99995, np.float32)
    theta = np.linspace(0.03, np.pi * 0.97, C).astype(np.float32)
    tr, ti = radius * np.cos(theta), radius * np.sin(theta)
    gm = np.sqrt(np.maximum(1 - radius ** 2, 1e-4)).astype(np.float32)
    raw = (rng.standard_normal((B, L, 3 * C)) * 8.0).astype(np.float32)
    raw[:, 40:80] = 0.0
    raw[:, 100:140, 2 * C:] = -60
    raw[:, 140:180, 2 * C:] = 60
    grad = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    read, state = emu.forward(raw, tr, ti, gm)
    want_read, want_state = field_oracle.forward(raw, tr, ti, gm)
    assert rel_err(read, want_read) < FP32_TOL
    assert rel_err(state, want_state) < FP32_TOL
    got = emu.backward(raw, tr, ti, gm, read, grad)
    want = field_oracle.backward(raw, tr, ti, gm, grad)
    for g, w in zip(got[:4], want[:4]):
        assert rel_err(g, w) < FP32_TOL


def test_decode_steps_continue_a_prefix():
    """Prefix in one pass, then token-by-token steps == one pass over prefix + tokens (causality)."""
    rng = np.random.default_rng(8)
    B, L, C, K = 3, 40, 12, 5
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L + K, 3 * C)).astype(np.float32)
    full, _ = field_oracle.forward(raw, tr, ti, gm)
    _, state = emu.forward(raw[:, :L], tr, ti, gm)
    for k in range(K):
        row, state = emu.step(raw[:, L + k], tr, ti, gm, state)
        assert rel_err(row, full[:, L + k]) < FP32_TOL
        assert rel_err(state, full[:, L + k, :2 * C]) < FP32_TOL


def test_decode_step_bf16_io():
    import torch
    rng = np.random.default_rng(9)
    B, C = 4, 16
    tr, ti, gm = _params(C, rng)
    raw = torch.from_numpy(rng.standard_normal((B, 3 * C)).astype(np.float32)).bfloat16()
    state = rng.standard_normal((B, 2 * C)).astype(np.float32)
    bits = raw.view(torch.int16).numpy().view(np.uint16)
    row_bits, new_state = emu.step(bits, tr, ti, gm, state, bf16=True)
    ref, ref_state = field_oracle.forward(raw.float().numpy()[:, None], tr, ti, gm, state_in=state)
    got = torch.from_numpy(np.array(row_bits).view(np.int16)).view(torch.bfloat16).float().numpy()
    assert rel_err(new_state, ref_state) < FP32_TOL          # the state never leaves fp32
    assert rel_err(got, ref[:, 0]) < 2 ** -8                 # one bf16 rounding of the output


def test_wait_selftest_reports_timeout():
    ws = emu._aligned(16384)
    assert emu.lib().fields_read_selftest_wait(ws.ctypes.data_as(emu.P), ws.size, 100, None) == 4
    assert emu.lib().fields_read_selftest_wait(ws.ctypes.data_as(emu.P), 64, 100, None) == 2


def _bits(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).bfloat16().view(torch.int16).numpy().view(np.uint16)


def _unbits(b):
    import torch
    return torch.from_numpy(np.array(b).view(np.int16)).view(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("B,L,C", [(2, 100, 132), (1, 37, 8), (1, 200, 512)])
def test_bf16_boundary_forward_backward(B, L, C):
    """bfloat16 raw / read / gradients, fp32 state: one bf16 rounding on outputs, and the
    2e-2 bound on gradients (s_{t-1} is read back from the bf16 forward output)."""
    from conftest import BF16_TOL
    rng = np.random.default_rng(B + L + C)
    tr, ti, gm = _params(C, rng)
    raw_b = _bits(rng.standard_normal((B, L, 3 * C)))
    grad_b = _bits(rng.standard_normal((B, L, 4 * C)))
    raw, grad = _unbits(raw_b), _unbits(grad_b)
    ref_read, _ = field_oracle.forward(raw, tr, ti, gm)
    read_b = emu.forward_bf16(raw_b, tr, ti, gm)
    assert rel_err(_unbits(read_b), ref_read) < 2 ** -7
    ref = field_oracle.backward(raw, tr, ti, gm, grad)
    got = emu.backward_bf16(raw_b, tr, ti, gm, read_b, grad_b)
    assert rel_err(_unbits(got[0]), ref[0]) < BF16_TOL
    for k in (1, 2, 3):
        assert rel_err(got[k], ref[k]) < BF16_TOL


@pytest.mark.parametrize("B,L,C", [(2, 130, 20), (1, 50, 512), (2, 7, 132)])
@pytest.mark.parametrize("order", ["forward", "reverse"])
def test_forward_with_norm_statistics(monkeypatch, B, L, C, order):
    """The per-token sums of squares that come with the bf16 forward equal those of the fp32
    oracle output, group by group, and `read` is the plain bf16 forward's."""
    monkeypatch.setenv("FIELDS_EMU_ORDER", order)
    rng = np.random.default_rng(B + L + C)
    tr, ti, gm = _params(C, rng)
    raw_b = _bits(rng.standard_normal((B, L, 3 * C)))
    ref_read, _ = field_oracle.forward(_unbits(raw_b), tr, ti, gm)
    read_b, sumsq = emu.forward_bf16_stats(raw_b, tr, ti, gm)
    np.testing.assert_array_equal(np.array(read_b), np.array(emu.forward_bf16(raw_b, tr, ti, gm)))
    G = (C + 127) // 128
    planes = ref_read.reshape(B, L, 4, C)
    want = np.stack([(planes[..., g * 128:(g + 1) * 128] ** 2).sum(axis=(2, 3)) for g in range(G)], -1)
    assert sumsq.shape == (B, L, G)
    assert rel_err(sumsq, want) < FP32_TOL


def test_bf16_boundary_refuses_odd_channel_counts():
    raw_b = np.zeros((1, 4, 21), np.uint16)
    p = np.ones(7, np.float32)
    with pytest.raises(RuntimeError, match="unsupported"):
        emu.forward_bf16(raw_b, p, p, p)


def test_mailbox_exchange_three_ranks_two_epochs():
    """Peer-memory exchange, emulated: every 'rank' puts its span summary into all mailboxes, then
    folds from its own; a second exchange on the other parity does not disturb the first; a
    mailbox that misses a summary reports the timeout."""
    rng = np.random.default_rng(12)
    B, L, C, world = 2, 90, 20, 3
    tr, ti, gm = _params(C, rng)
    boxes = emu.make_mailboxes(world, B, C)
    for epoch in (1, 2, 3):
        raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
        s0 = rng.standard_normal((B, 2 * C)).astype(np.float32)
        cuts = [0, 31, 64, L]
        spans = [raw[:, a:b] for a, b in zip(cuts[:-1], cuts[1:])]
        for r, x in enumerate(spans):
            got = emu.span_summary_put(x, tr, ti, gm, boxes, r, epoch)
            assert rel_err(got, field_oracle.span_summary(x, tr, ti, gm)) < FP32_TOL
        state = s0.astype(np.float64)
        for r, x in enumerate(spans):
            got, err = emu.fold_mailbox(boxes[r], r, world, epoch, B, C, state0=s0)
            assert err == 0
            assert rel_err(got, state) < FP32_TOL
            _, state = field_oracle.forward(x, tr, ti, gm, state_in=state)
    # an exchange in which rank 1 never puts: everyone's wait runs out (at once in the emulation)
    fresh = emu.make_mailboxes(world, B, C)
    for r in (0, 2):
        emu.span_summary_put(spans[r], tr, ti, gm, fresh, r, 1)
    got, err = emu.fold_mailbox(fresh[2], 2, world, 1, B, C)
    assert err == 1 and np.isnan(got).all()


def test_mailbox_exchange_carries_the_backward_too():
    """Forward and backward exchanges alternate on the same mailboxes (epochs 1, 2, 3, 4): the
    carries folded from the mailboxes equal those folded from gathered dual summaries."""
    rng = np.random.default_rng(21)
    B, L, C, world = 2, 90, 20, 3
    tr, ti, gm = _params(C, rng)
    boxes = emu.make_mailboxes(world, B, C)
    cuts = [0, 31, 64, L]
    epoch = 0
    for _ in range(2):
        raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
        grad = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
        g_end = rng.standard_normal((B, 2 * C)).astype(np.float32)
        spans = list(zip(cuts[:-1], cuts[1:]))
        epoch += 1
        for r, (a, b) in enumerate(spans):
            emu.span_summary_put(raw[:, a:b], tr, ti, gm, boxes, r, epoch)
        states = [emu.fold_mailbox(boxes[r], r, world, epoch, B, C)[0] for r in range(world)]
        epoch += 1
        dual = np.stack([emu.span_summary_backward_put(raw[:, a:b], tr, ti, grad[:, a:b], boxes, r, epoch)
                         for r, (a, b) in enumerate(spans)])
        for r in range(world):
            got, err = emu.fold_mailbox_backward(boxes[r], r, world, epoch, B, C, carry_end=g_end)
            assert err == 0
            np.testing.assert_allclose(got, emu.fold_summaries_backward(dual, r, carry_end=g_end),
                                       rtol=1e-6, atol=1e-7)
        # the forward states of this round are untouched by the backward exchange on the other parity
        want = np.zeros((B, 2 * C))
        for r, (a, b) in enumerate(spans):
            assert rel_err(states[r], want) < FP32_TOL or r == 0
            _, want = field_oracle.forward(raw[:, a:b], tr, ti, gm, state_in=want)


def test_sum_over_ranks_through_the_mailboxes():
    """The parameter-gradient sum of a sharded backward pass without a collective library: every
    rank stores its addends into all mailboxes and adds what arrived in rank order, so all ranks
    hold the same bits; the exchange shares mailboxes and epochs with the summary exchanges; a
    rank that never stores makes the others report the timeout."""
    rng = np.random.default_rng(33)
    B, C, world = 2, 20, 3
    tr, ti, gm = _params(C, rng)
    boxes = emu.make_mailboxes(world, B, C)
    n = 3 * C + 1
    raw = rng.standard_normal((B, 12, 3 * C)).astype(np.float32)
    for epoch in (1, 2, 3, 4):
        if epoch == 2:   # a summary exchange in between, on the same mailboxes
            for r in range(world):
                emu.span_summary_put(raw, tr, ti, gm, boxes, r, epoch)
            continue
        vals = [rng.standard_normal(n).astype(np.float32) for _ in range(world)]
        outs, errs = emu.sum_over_ranks(vals, boxes, epoch, B, C)
        want = (vals[0] + vals[1]) + vals[2]          # rank order, fp32
        assert errs == [0, 0, 0]
        for out in outs:
            np.testing.assert_array_equal(out, want)
    vals = [rng.standard_normal(n).astype(np.float32) for _ in range(world)]
    outs, errs = emu.sum_over_ranks(vals, boxes, 5, B, C, absent=(1,))
    assert errs[0] == 1 and errs[2] == 1 and np.isnan(outs[0]).all() and np.isnan(outs[2]).all()
    lib = emu.lib()
    ptrs = (emu.ctypes.c_void_p * world)(*[m.ctypes.data for m in boxes])
    v = emu._f32(np.zeros(3 * C + 65))
    err = np.zeros(1, dtype=np.uint32)
    args = (emu._ptr(v), emu._ptr(v))
    assert lib.fields_read_sum_over_ranks(*args, 3 * C + 65, ptrs, emu._ptr(err), 0, world, 1, 0, B, C, None) == 1
    assert lib.fields_read_sum_over_ranks(*args, 4, ptrs, emu._ptr(err), 0, world, 0, 0, B, C, None) == 1
    assert lib.fields_read_sum_over_ranks(*args, 4, ptrs, emu._ptr(err), 3, world, 1, 0, B, C, None) == 1
    assert lib.fields_read_sum_over_ranks(*args, 0, ptrs, emu._ptr(err), 0, world, 1, 0, B, C, None) == 0


@pytest.mark.parametrize("B,L,C,cuts", [
    (1, 700, 512, [0, 233, 480, 700]),     # four chains, several runs per chain, ragged spans
    (2, 90, 20, [0, 31, 64, 90]),          # one partly filled channel group
    (3, 130, 132, [0, 130]),               # a single rank: nothing is exchanged
    (9, 61, 260, [0, 7, 61]),              # more chains than blocks: several items per block
])
def test_sharded_forward_in_one_launch(B, L, C, cuts):
    """fields_read_forward_sharded, emulated: every rank sweeps its span and stores its map into
    all mailboxes, then every rank waits, folds and sweeps again. `read`, the span maps and the
    end states equal the oracle's full-sequence pass; two calls alternate the mailbox parities."""
    rng = np.random.default_rng(B * 1000 + L + C)
    tr, ti, gm = _params(C, rng)
    world = len(cuts) - 1
    boxes = emu.make_mailboxes(world, B, C)
    for epoch in (1, 2, 3):
        raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
        s0 = rng.standard_normal((B, 2 * C)).astype(np.float32) if epoch != 2 else None
        ranks = [emu.ShardedForward(raw[:, a:b], tr, ti, gm, boxes, r, state0=s0)
                 for r, (a, b) in enumerate(zip(cuts[:-1], cuts[1:]))]
        for stage in (1, 4, 2):     # all first sweeps, all sends, then the waits and second sweeps
            for op in ranks:
                op.run(stage, epoch)
        want_read, _ = field_oracle.forward(raw, tr, ti, gm, state_in=s0)
        got = np.concatenate([op.read for op in ranks], axis=1)
        assert rel_err(got, want_read) < FP32_TOL
        state = None if s0 is None else s0.astype(np.float64)
        for op, (a, b) in zip(ranks, zip(cuts[:-1], cuts[1:])):
            assert int(op.err[0]) == 0
            assert rel_err(op.summary, field_oracle.span_summary(raw[:, a:b], tr, ti, gm)) < FP32_TOL
            _, state = field_oracle.forward(raw[:, a:b], tr, ti, gm, state_in=state)
            assert rel_err(op.state, state) < FP32_TOL


def test_sharded_forward_reports_a_missing_summary():
    """A rank whose peer never ran: the wait runs out (at once in the emulation), the error word
    is set and the outputs hold NaN; the rank before it is unaffected in its own arithmetic."""
    rng = np.random.default_rng(77)
    B, L, C = 1, 200, 128
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    boxes = emu.make_mailboxes(2, B, C)
    late = emu.ShardedForward(raw[:, 100:], tr, ti, gm, boxes, 1)
    for stage in (1, 4, 2):  # rank 0 never stored its summary
        late.run(stage, 1)
    assert int(late.err[0]) == 1 and np.isnan(late.read).all() and np.isnan(late.state).all()


@pytest.mark.parametrize("B,L,C", [(1, 300, 32), (2, 130, 20), (1, 128, 64), (2, 17, 36)])
def test_tensor_core_formulation_of_the_forward(B, L, C):
    """The prefix-ratio restatement (sub-chunks of 16 steps, quotients b / P rounded to bfloat16,
    summed by a triangular all-ones matrix) with the contraction emulated over the operand
    layouts the tensor cores read: within the bfloat16 tolerance of the oracle, including
    saturated vacancy gates (|a| at its minimum, where 1 / |P| is largest)."""
    rng = np.random.default_rng(B * 100 + L + C)
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    raw[:, L // 3: L // 3 + 40, 2 * C:] = 30.0      # vacancy saturated for a stretch
    raw_b = _bits(raw)
    s0 = rng.standard_normal((B, 2 * C)).astype(np.float32)
    ref_read, ref_state = field_oracle.forward(_unbits(raw_b), tr, ti, gm, state_in=s0)
    read_b, state, err = emu.forward_bf16_tensor(raw_b, tr, ti, gm, state_in=s0)
    assert err == 0
    assert rel_err(_unbits(read_b), ref_read) < BF16_TOL
    assert rel_err(state, ref_state) < BF16_TOL
