"""Sequence-sharded forward on real GPUs (needs at least two): every rank's span must equal the
corresponding slice of a single-GPU full-sequence pass and of the CPU oracle."""
import datetime
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, L, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=90))
    problems = []   # checked only after every rank's kernels are done and the ranks have met

    def check(ok, what):
        if not ok:
            problems.append(f"rank {rank}: {what}")
    try:
        from fields_lm_b200 import field_read_with_state, seqpar
        gen = torch.Generator().manual_seed(123)
        B, C = 1, 512
        ring = torch.linspace(0.85, 0.999, C)
        theta = torch.linspace(0.03, torch.pi * 0.97, C)
        tr, ti = (ring * torch.cos(theta)).to(dev), (ring * torch.sin(theta)).to(dev)
        gm = torch.sqrt(1 - ring ** 2).to(dev)
        raw = (torch.randn(B, L, 3 * C, generator=gen) * 0.577)
        lo, hi = seqpar.span_bounds(L, world, rank)
        span = raw[:, lo:hi].contiguous().to(dev)
        read, state = seqpar.sequence_parallel_field_read(span, tr, ti, gm)
        torch.cuda.synchronize()
        # the preallocated form gives the same bits, call after call
        op = seqpar.SequenceParallelForward(B, hi - lo, C, dev)
        for _ in range(2):
            read2, state2 = op(span, tr, ti, gm)
        torch.cuda.synchronize()
        check(float((read2 - read).abs().max()) <= 2e-6 * float(read.abs().max()), "NCCL read")
        check(float((state2 - state).abs().max()) <= 2e-6 * float(state.abs().max()), "NCCL state")
        # the same exchange through peer memory instead of NCCL; several calls alternate parities
        p2p = seqpar.SequenceParallelForwardP2P(B, hi - lo, C, dev)
        for _ in range(3):
            read3, state3 = p2p(span, tr, ti, gm)
        torch.cuda.synchronize()
        check(p2p.status() == 0, "peer-memory exchange timed out")
        check(float((read3 - read).abs().max()) <= 2e-6 * float(read.abs().max()), "P2P read")
        check(float((state3 - state).abs().max()) <= 2e-6 * float(state.abs().max()), "P2P state")
        # the whole sharded forward as one cooperative launch per rank
        fused = seqpar.SequenceParallelForwardFused(B, hi - lo, C, dev)
        for _ in range(4):
            read4, state4 = fused(span, tr, ti, gm)
        torch.cuda.synchronize()
        # the same with the epoch kept on the device (the form a captured graph can replay)
        fused_dev = seqpar.SequenceParallelForwardFused(B, hi - lo, C, dev, device_epoch=True)
        for _ in range(4):
            read5, state5 = fused_dev(span, tr, ti, gm)
        torch.cuda.synchronize()
        check(fused_dev.status() == 0, "one-launch forward with a device epoch timed out")
        check(float((read5 - read).abs().max()) <= 2e-6 * float(read.abs().max()), "device-epoch read")
        check(float((state5 - state).abs().max()) <= 2e-6 * float(state.abs().max()), "device-epoch state")
        check(fused.status() == 0, "one-launch forward timed out")
        check(float((read4 - read).abs().max()) <= 2e-6 * float(read.abs().max()), "fused read")
        check(float((state4 - state).abs().max()) <= 2e-6 * float(state.abs().max()), "fused state")
        if rank == 0:
            with torch.no_grad():
                full, full_state = field_read_with_state(raw.to(dev), tr, ti, gm, None)
            np.savez(os.path.join(out_dir, "full.npz"), read=full.cpu().numpy(),
                     state=full_state.cpu().numpy(), raw=raw.numpy(), tr=tr.cpu().numpy(),
                     ti=ti.cpu().numpy(), gm=gm.cpu().numpy())
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), read=read.cpu().numpy(),
                 state=state.cpu().numpy(), lo=lo, hi=hi)
        # every rank leaves in order, with nothing in flight, also when a check failed
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()
    assert not problems, problems


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("L", [4096, 16384 + 37])
def test_sequence_sharded_forward_matches_single_gpu_and_oracle(tmp_path, L):
    import torch.multiprocessing as mp
    from conftest import FP32_TOL, rel_err
    from oracle import field_oracle
    world = torch.cuda.device_count()
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, L, str(tmp_path)), nprocs=world, join=True)
    full = np.load(tmp_path / "full.npz")
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    got = np.concatenate([p["read"] for p in parts], axis=1)
    assert rel_err(got, full["read"]) < 2e-6
    ref, ref_state = field_oracle.forward(full["raw"], full["tr"], full["ti"], full["gm"])
    assert rel_err(got, ref) < FP32_TOL
    assert rel_err(parts[-1]["state"], ref_state) < FP32_TOL


def _train_worker(rank, world, port, L, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=90))
    problems = []   # checked only after every rank's kernels are done and the ranks have met

    def check(ok, what):
        if not ok:
            problems.append(f"rank {rank}: {what}")
    try:
        from fields_lm_b200 import seqpar
        gen = torch.Generator().manual_seed(321)
        B, C = 2, 512
        ring = torch.linspace(0.85, 0.999, C)
        theta = torch.linspace(0.03, torch.pi * 0.97, C)
        tr = (ring * torch.cos(theta)).to(dev).requires_grad_(True)
        ti = (ring * torch.sin(theta)).to(dev).requires_grad_(True)
        gm = torch.sqrt(1 - ring ** 2).to(dev).requires_grad_(True)
        raw = torch.randn(B, L, 3 * C, generator=gen) * 0.577
        grad = torch.randn(B, L, 4 * C, generator=gen)
        lo, hi = seqpar.span_bounds(L, world, rank)
        span = raw[:, lo:hi].contiguous().to(dev).requires_grad_(True)
        read = seqpar.sequence_parallel_field_read_autograd(span, tr, ti, gm)
        read.backward(grad[:, lo:hi].contiguous().to(dev))
        torch.cuda.synchronize()
        # the same step on preallocated buffers
        step = seqpar.SequenceParallelTrainStep(B, hi - lo, C, dev)
        g_span = grad[:, lo:hi].contiguous().to(dev)
        for _ in range(2):
            step.forward(span.detach(), tr.detach(), ti.detach(), gm.detach())
            g_raw, g_par = step.backward(span.detach(), tr.detach(), ti.detach(), gm.detach(), g_span)
        torch.cuda.synchronize()
        check(float((g_raw - span.grad).abs().max()) <= 1e-5 * float(span.grad.abs().max()), "NCCL grad_raw")
        for k, t in enumerate((tr, ti, gm)):
            check(float((g_par[k] - t.grad).abs().max()) <= 1e-5 * float(t.grad.abs().max()),
                  f"NCCL parameter gradient {k}")
        # and with both exchanges through peer memory
        p2p = seqpar.SequenceParallelTrainStepP2P(B, hi - lo, C, dev)
        for _ in range(3):
            p2p.forward(span.detach(), tr.detach(), ti.detach(), gm.detach())
            g_raw2, g_par2 = p2p.backward(span.detach(), tr.detach(), ti.detach(), gm.detach(), g_span)
        torch.cuda.synchronize()
        check(p2p.status() == 0, "peer-memory exchange timed out")
        check(float((g_raw2 - span.grad).abs().max()) <= 1e-5 * float(span.grad.abs().max()), "P2P grad_raw")
        for k, t in enumerate((tr, ti, gm)):
            check(float((g_par2[k] - t.grad).abs().max()) <= 1e-5 * float(t.grad.abs().max()),
                  f"P2P parameter gradient {k}")
        if rank == 0:
            np.savez(os.path.join(out_dir, "inputs.npz"), raw=raw.numpy(), grad=grad.numpy(),
                     tr=tr.detach().cpu().numpy(), ti=ti.detach().cpu().numpy(),
                     gm=gm.detach().cpu().numpy())
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), lo=lo, hi=hi,
                 grad_raw=span.grad.cpu().numpy(), grad_tr=tr.grad.cpu().numpy(),
                 grad_ti=ti.grad.cpu().numpy(), grad_gamma=gm.grad.cpu().numpy())
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()
    assert not problems, problems


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_sequence_sharded_training_step_matches_the_oracle(tmp_path):
    """Forward + backward of a sequence sharded over the GPUs: gradients of every span and the
    all-reduced parameter gradients equal the single-device ones."""
    import torch.multiprocessing as mp
    from conftest import FP32_TOL, rel_err
    from oracle import field_oracle
    L = 2048 + 11
    world = torch.cuda.device_count()
    port = 30600 + (os.getpid() % 2000)
    mp.spawn(_train_worker, args=(world, port, L, str(tmp_path)), nprocs=world, join=True)
    x = np.load(tmp_path / "inputs.npz")
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    want = field_oracle.backward(x["raw"], x["tr"], x["ti"], x["gm"], x["grad"])
    assert rel_err(np.concatenate([p["grad_raw"] for p in parts], axis=1), want[0]) < FP32_TOL
    for k, name in enumerate(("grad_tr", "grad_ti", "grad_gamma")):
        for p in parts:
            assert rel_err(p[name], want[1 + k]) < FP32_TOL
