"""``fields_read_forward_sharded`` on ONE GPU, through the C ABI.

The sequence-sharded forward of one rank as a single cooperative launch. With P = 1 nothing is
exchanged, so one GPU checks the two sweeps, the in-kernel scan and the run bookkeeping against
the CPU oracle; the mailbox protocol between ranks is checked on several GPUs
(``test_gpu_seqpar.py``) and, rank by rank, in the host emulation. A second rank that never
shows up makes the bounded wait run out: the call must come back with the error word set.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import FP32_TOL, rel_err
from oracle import field_oracle

pytestmark = pytest.mark.gpu


def _params(C, rng):
    radius = rng.uniform(0.5, 0.99995, C).astype(np.float32)
    theta = rng.uniform(-np.pi, np.pi, C).astype(np.float32)
    return ((radius * np.cos(theta)).astype(np.float32),
            (radius * np.sin(theta)).astype(np.float32),
            np.sqrt(np.maximum(1 - radius ** 2, 1e-4)).astype(np.float32))


class Rank:
    """Buffers of one rank of a P-rank job whose other ranks do not exist."""

    def __init__(self, dev, B, L, C, P=1, rank=0):
        from fields_lm_b200 import _lib
        self.lib = _lib.load()
        self.dims = (B, L, C)
        self.P, self.rank = P, rank
        self.read = torch.full((B, L, 4 * C), float("nan"), device=dev)
        self.state = torch.full((B, 2 * C), float("nan"), device=dev)
        self.summary = torch.full((B, 4, C), float("nan"), device=dev)
        n = self.lib.fields_read_mailbox_bytes(P, B, C)
        self.mail = [torch.zeros(n, dtype=torch.uint8, device=dev) for _ in range(P)]
        self.peers = (ctypes.c_void_p * P)(*[m.data_ptr() for m in self.mail])
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.stream = torch.cuda.current_stream(dev).cuda_stream

    def __call__(self, raw, tr, ti, gm, epoch, state0=None, max_polls=0):
        B, L, C = self.dims
        return self.lib.fields_read_forward_sharded(
            raw.data_ptr(), tr.data_ptr(), ti.data_ptr(), gm.data_ptr(),
            None if state0 is None else state0.data_ptr(), self.read.data_ptr(),
            self.state.data_ptr(), self.summary.data_ptr(), self.peers, self.err.data_ptr(),
            self.rank, self.P, epoch, max_polls, B, L, C, self.stream)


@pytest.mark.parametrize("B,L,C", [(1, 8192, 512), (2, 1000, 512), (3, 37, 20), (1, 1, 4),
                                   (5, 300, 132), (40, 130, 512), (1, 48 * 74 + 5, 512)])
def test_single_rank_matches_the_oracle(B, L, C):
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(B * 7 + L + C)
    tr, ti, gm = _params(C, rng)
    op = Rank(dev, B, L, C)
    t = [torch.from_numpy(a).to(dev) for a in (tr, ti, gm)]
    for epoch in (1, 2, 3):
        raw = (rng.standard_normal((B, L, 3 * C)) * (1.0 if epoch < 3 else 3.0)).astype(np.float32)
        s0 = rng.standard_normal((B, 2 * C)).astype(np.float32) if epoch != 2 else None
        s0_t = None if s0 is None else torch.from_numpy(s0).to(dev)
        assert op(torch.from_numpy(raw).to(dev), *t, epoch, state0=s0_t) == 0
        torch.cuda.synchronize()
        assert int(op.err.item()) == 0
        want_read, want_state = field_oracle.forward(raw, tr, ti, gm, state_in=s0)
        assert rel_err(op.read.cpu().numpy(), want_read) < FP32_TOL
        assert rel_err(op.state.cpu().numpy(), want_state) < FP32_TOL
        assert rel_err(op.summary.cpu().numpy(), field_oracle.span_summary(raw, tr, ti, gm)) < FP32_TOL


def test_equals_the_plain_forward_at_the_sharded_span_size():
    """8,192 tokens x 512 channels (one rank's span of the 65,536-token forward at 8 ranks)."""
    from fields_lm_b200 import field_read_with_state
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(2)
    B, L, C = 1, 8192, 512
    ring = torch.linspace(0.85, 0.999, C)
    theta = torch.linspace(0.03, torch.pi * 0.97, C)
    t = [(ring * torch.cos(theta)).to(dev), (ring * torch.sin(theta)).to(dev),
         torch.sqrt(1 - ring ** 2).to(dev)]
    raw = (torch.randn(B, L, 3 * C, generator=gen) * 0.577).bfloat16().float().to(dev)
    op = Rank(dev, B, L, C)
    for epoch in range(1, 6):
        assert op(raw, *t, epoch) == 0
    with torch.no_grad():
        want, want_state = field_read_with_state(raw, *t, None)
    torch.cuda.synchronize()
    assert int(op.err.item()) == 0
    assert rel_err(op.read.cpu().numpy(), want.cpu().numpy()) < 2e-6
    assert rel_err(op.state.cpu().numpy(), want_state.cpu().numpy()) < 2e-6


def test_an_absent_peer_ends_the_wait_with_the_error_word_set():
    """Rank 1 of 2, and rank 0 never runs: the wait for its summary is bounded (2,000 polls
    here), the kernel ends, the error word is 1 and the outputs hold NaN. Nothing hangs, traps or
    faults; the next ordinary call works."""
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(5)
    B, L, C = 1, 600, 512
    tr, ti, gm = _params(C, rng)
    t = [torch.from_numpy(a).to(dev) for a in (tr, ti, gm)]
    raw = torch.from_numpy(rng.standard_normal((B, L, 3 * C)).astype(np.float32)).to(dev)
    op = Rank(dev, B, L, C, P=2, rank=1)
    assert op(raw, *t, 1, max_polls=2000) == 0
    torch.cuda.synchronize()
    assert int(op.err.item()) == 1
    assert bool(torch.isnan(op.read).all()) and bool(torch.isnan(op.state).all())
    # the span's own map was still computed and stored, in its own mailbox too
    assert rel_err(op.summary.cpu().numpy(),
                   field_oracle.span_summary(raw.cpu().numpy(), tr, ti, gm)) < FP32_TOL
    solo = Rank(dev, B, L, C)
    assert solo(raw, *t, 1) == 0
    torch.cuda.synchronize()
    assert int(solo.err.item()) == 0 and bool(torch.isfinite(solo.read).all())


def test_device_epoch_calls_and_cuda_graph_replay():
    """epoch 0: the epoch lives on the rank's board and the kernel advances it, so the same call
    can be issued again and again, directly and replayed from a captured CUDA graph (with new
    data in the same buffers each time)."""
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(9)
    B, L, C = 2, 3000, 512
    tr, ti, gm = _params(C, rng)
    t = [torch.from_numpy(a).to(dev) for a in (tr, ti, gm)]
    op = Rank(dev, B, L, C)
    raw = torch.empty(B, L, 3 * C, device=dev)

    def fresh():
        data = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
        raw.copy_(torch.from_numpy(data))
        return data

    def check(data):
        torch.cuda.synchronize()
        want, want_state = field_oracle.forward(data, tr, ti, gm)
        assert int(op.err.item()) == 0
        assert rel_err(op.read.cpu().numpy(), want) < FP32_TOL
        assert rel_err(op.state.cpu().numpy(), want_state) < FP32_TOL

    for _ in range(3):                       # direct calls, epochs 1, 2, 3 kept on the device
        data = fresh()
        assert op(raw, *t, 0) == 0
        check(data)
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        op.stream = side.cuda_stream
        assert op(raw, *t, 0) == 0           # warm-up on the capture stream
        with torch.cuda.graph(graph, stream=side):
            assert op(raw, *t, 0) == 0
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize()
    for _ in range(4):
        data = fresh()
        graph.replay()
        check(data)


def test_sum_over_ranks_alone_and_with_an_absent_peer():
    """fields_read_sum_over_ranks on one GPU: with P = 1 the sum is the rank's own vector; as rank
    1 of 2 whose peer never stores, the bounded wait ends with the error word set and NaN in the
    result (nothing hangs), and the mailbox works again under the next epoch."""
    from fields_lm_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, C = 1, 512
    n = 3 * C + 1
    st = torch.cuda.current_stream(dev).cuda_stream
    vals = torch.randn(n, device=dev)
    out = torch.full((n,), float("nan"), device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)

    def boxes(P):
        size = lib.fields_read_mailbox_bytes(P, B, C)
        mail = [torch.zeros(size, dtype=torch.uint8, device=dev) for _ in range(P)]
        return mail, (ctypes.c_void_p * P)(*[m.data_ptr() for m in mail])

    mail, ptrs = boxes(1)
    for epoch in (1, 2, 3):
        vals.normal_()
        assert lib.fields_read_sum_over_ranks(vals.data_ptr(), out.data_ptr(), n, ptrs, err.data_ptr(),
                                              0, 1, epoch, 0, B, C, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, vals) and int(err.item()) == 0
    mail2, ptrs2 = boxes(2)
    assert lib.fields_read_sum_over_ranks(vals.data_ptr(), out.data_ptr(), n, ptrs2, err.data_ptr(),
                                          1, 2, 1, 2000, B, C, st) == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 1 and bool(torch.isnan(out).all())
    # both ranks of the next epoch, played by this GPU one after the other: rank 0 stores and
    # gives up (its peer has not stored yet), then rank 1 finds both contributions
    err.zero_()
    other = torch.randn(n, device=dev)
    scratch = torch.empty(n, device=dev)
    lib.fields_read_sum_over_ranks(other.data_ptr(), scratch.data_ptr(), n, ptrs2, err.data_ptr(),
                                   0, 2, 2, 50, B, C, st)
    err.zero_()
    assert lib.fields_read_sum_over_ranks(vals.data_ptr(), out.data_ptr(), n, ptrs2, err.data_ptr(),
                                          1, 2, 2, 0, B, C, st) == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 0 and torch.equal(out, other + vals)


def test_argument_errors():
    dev = torch.device("cuda", 0)
    op = Rank(dev, 1, 8, 4)
    p = torch.ones(4, device=dev)
    raw = torch.zeros(1, 8, 12, device=dev)
    op.rank = 1
    assert op(raw, p, p, p, 1) == 1                       # rank outside [0, P)
    odd = Rank(dev, 1, 8, 3)
    p3 = torch.ones(3, device=dev)
    assert odd(torch.zeros(1, 8, 9, device=dev), p3, p3, p3, 1) == 5   # C % 4 != 0


@pytest.mark.parametrize("backward", [False, True])
def test_fold_mailbox_gives_up_after_max_polls(backward):
    """The three-launch exchange's wait: a zeroed mailbox in which no summary ever arrives. With
    the bound set to 2,000 polls the call ends at once, sets the error word and writes NaN; one
    late slot ends the waiting for all that follow it (one bound per call, not per slot)."""
    import time
    from fields_lm_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    P, B, C = 8, 1, 512
    mail = torch.zeros(lib.fields_read_mailbox_bytes(P, B, C), dtype=torch.uint8, device=dev)
    state = torch.zeros(B, 2 * C, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    fn = lib.fields_read_fold_mailbox_backward if backward else lib.fields_read_fold_mailbox
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    assert fn(mail.data_ptr(), None, state.data_ptr(), err.data_ptr(), 3, P, 1, 2000, B, C,
              torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5      # 4 P slots x 2,000 polls each would take far longer
    assert int(err.item()) == 1 and bool(torch.isnan(state).all())
