"""Sequence-sharded forward and backward on CPU: gloo ranks, the device operations emulated on
the host.

Checks the host logic of fields_lm_b200.seqpar (span bounds, gather, fold order in both
directions, state and gradient-carry hand-over, parameter-gradient reduction) against a single
full-sequence pass of the oracle.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class EmuOps:
    """Same three operations as seqpar.CudaOps, through the host emulation of the CUDA source."""

    def span_summary(self, raw, tr, ti, gamma):
        import emu
        return torch.from_numpy(np.array(emu.span_summary(raw.numpy(), tr.numpy(), ti.numpy(),
                                                          gamma.numpy())))

    def fold(self, summaries, rank, state0):
        import emu
        s0 = None if state0 is None else state0.numpy()
        return torch.from_numpy(np.array(emu.fold_summaries(summaries.numpy(), rank, s0)))

    def forward(self, raw, tr, ti, gamma, state_in):
        import emu
        s_in = None if state_in is None else state_in.numpy()
        read, state = emu.forward(raw.numpy(), tr.numpy(), ti.numpy(), gamma.numpy(), state_in=s_in)
        return torch.from_numpy(np.array(read)), torch.from_numpy(np.array(state))


    def span_summary_backward(self, raw, tr, ti, grad_read):
        import emu
        return torch.from_numpy(np.array(emu.span_summary_backward(raw.numpy(), tr.numpy(),
                                                                   ti.numpy(), grad_read.numpy())))

    def fold_backward(self, summaries, rank, carry_end):
        import emu
        c = None if carry_end is None else carry_end.numpy()
        return torch.from_numpy(np.array(emu.fold_summaries_backward(summaries.numpy(), rank, c)))

    def backward(self, raw, tr, ti, gamma, read, grad_read, state_in, grad_state_out):
        import emu
        s_in = None if state_in is None else state_in.numpy()
        g_out = None if grad_state_out is None else grad_state_out.numpy()
        g_raw, g_tr, g_ti, g_gm, g_sin = emu.backward(raw.numpy(), tr.numpy(), ti.numpy(),
                                                      gamma.numpy(), read.numpy(), grad_read.numpy(),
                                                      state_in=s_in, grad_state_out=g_out)
        return (torch.from_numpy(np.array(g_raw)),
                torch.from_numpy(np.stack([np.array(g_tr), np.array(g_ti), np.array(g_gm)])),
                torch.from_numpy(np.array(g_sin)))


def _problem(L, with_state0):
    gen = torch.Generator().manual_seed(99)
    B, C = 2, 20
    radius = torch.rand(C, generator=gen) * 0.49 + 0.5
    theta = (torch.rand(C, generator=gen) * 2 - 1) * torch.pi
    tr, ti = radius * torch.cos(theta), radius * torch.sin(theta)
    gamma = torch.sqrt(1 - radius ** 2)
    raw = torch.randn(B, L, 3 * C, generator=gen)
    state0 = torch.randn(B, 2 * C, generator=gen) if with_state0 else None
    grad = torch.randn(B, L, 4 * C, generator=gen)
    return tr, ti, gamma, raw, state0, grad


def _train_worker(rank, world, port, L, with_state0, reduce, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fields_lm_b200 import seqpar
        tr, ti, gamma, raw, state0, grad = _problem(L, with_state0)
        lo, hi = seqpar.span_bounds(L, world, rank)
        span = raw[:, lo:hi].clone().requires_grad_(True)
        tr, ti, gamma = (t.clone().requires_grad_(True) for t in (tr, ti, gamma))
        read = seqpar.sequence_parallel_field_read_autograd(span, tr, ti, gamma, state0=state0,
                                                            ops=EmuOps(),
                                                            reduce_parameter_grads=reduce)
        (read * grad[:, lo:hi]).sum().backward()
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), lo=lo, hi=hi, read=read.detach().numpy(),
                 grad_raw=span.grad.numpy(), grad_tr=tr.grad.numpy(), grad_ti=ti.grad.numpy(),
                 grad_gamma=gamma.grad.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L,with_state0,reduce", [(2, 101, False, True), (3, 50, True, True),
                                                        (2, 64, True, False)])
def test_sharded_training_step_matches_one_device(tmp_path, world, L, with_state0, reduce):
    from conftest import FP32_TOL, rel_err
    from oracle import field_oracle
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_train_worker, args=(world, port, L, with_state0, reduce, str(tmp_path)), nprocs=world,
             join=True)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    tr, ti, gamma, raw, state0, grad = _problem(L, with_state0)
    s0 = None if state0 is None else state0.numpy()
    want = field_oracle.backward(raw.numpy(), tr.numpy(), ti.numpy(), gamma.numpy(), grad.numpy(),
                                 state_in=s0)
    ref_read, _ = field_oracle.forward(raw.numpy(), tr.numpy(), ti.numpy(), gamma.numpy(), state_in=s0)
    assert rel_err(np.concatenate([p["read"] for p in parts], axis=1), ref_read) < FP32_TOL
    assert rel_err(np.concatenate([p["grad_raw"] for p in parts], axis=1), want[0]) < FP32_TOL
    for k, name in enumerate(("grad_tr", "grad_ti", "grad_gamma")):
        if reduce:  # every rank holds the full gradient
            for p in parts:
                assert rel_err(p[name], want[1 + k]) < FP32_TOL
        else:       # each rank holds its span's share
            assert rel_err(sum(p[name].astype(np.float64) for p in parts), want[1 + k]) < FP32_TOL


def _worker(rank, world, port, L, with_state0, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fields_lm_b200 import seqpar
        gen = torch.Generator().manual_seed(99)
        B, C = 2, 20
        radius = torch.rand(C, generator=gen) * 0.49 + 0.5
        theta = (torch.rand(C, generator=gen) * 2 - 1) * torch.pi
        tr, ti = radius * torch.cos(theta), radius * torch.sin(theta)
        gamma = torch.sqrt(1 - radius ** 2)
        raw = torch.randn(B, L, 3 * C, generator=gen)
        state0 = torch.randn(B, 2 * C, generator=gen) if with_state0 else None
        lo, hi = seqpar.span_bounds(L, world, rank)
        read, state = seqpar.sequence_parallel_field_read(raw[:, lo:hi], tr, ti, gamma,
                                                          state0=state0, ops=EmuOps())
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), read=read.numpy(), state=state.numpy(),
                 lo=lo, hi=hi, raw=raw.numpy(), tr=tr.numpy(), ti=ti.numpy(), gamma=gamma.numpy(),
                 state0=np.zeros(0) if state0 is None else state0.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L,with_state0", [(2, 101, False), (2, 64, True), (3, 50, True)])
def test_spans_reassemble_to_the_full_sequence(tmp_path, world, L, with_state0):
    from conftest import FP32_TOL, rel_err
    from oracle import field_oracle
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, L, with_state0, str(tmp_path)), nprocs=world, join=True)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    p0 = parts[0]
    s0 = p0["state0"] if p0["state0"].size else None
    ref, ref_state = field_oracle.forward(p0["raw"], p0["tr"], p0["ti"], p0["gamma"], state_in=s0)
    assert [int(p["lo"]) for p in parts][0] == 0 and int(parts[-1]["hi"]) == L
    got = np.concatenate([p["read"] for p in parts], axis=1)
    assert rel_err(got, ref) < FP32_TOL
    assert rel_err(parts[-1]["state"], ref_state) < FP32_TOL


def test_span_bounds_cover_the_sequence():
    from fields_lm_b200.seqpar import span_bounds
    for L, P in [(65536, 8), (10, 3), (7, 7), (100, 1)]:
        cuts = [span_bounds(L, P, r) for r in range(P)]
        assert cuts[0][0] == 0 and cuts[-1][1] == L
        assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
        assert max(hi - lo for lo, hi in cuts) - min(hi - lo for lo, hi in cuts) <= 1
