#!/usr/bin/env python
"""Benchmark of the Field-recurrence operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward + backward pass of the fused Field read over one batch of
synthetic input: batch 8 x 2,048 tokens, d_model 1024 (C = 512 complex channels),
bf16-rounded activations held in fp32 at the operator boundary, fp32 state.
Under torchrun every rank runs that workload on its own GPU (batch-sharded,
no collective on the data path; weak scaling); rank 0 prints ONE JSON line.

`value` is tokens/s with inputs resident in HBM, through the C ABI on preallocated
buffers, timed with CUDA events on the launching stream; `e2e` is the same metric from pinned host buffers through the
public Python call and back to the host; `roofline` relates the step to the
measured HBM copy bandwidth; `cpu_baseline` times the reference's own CPU implementation
(`reference_field_read` + autograd, from the staged copy under oracle/_ref) on the host cores
(a reported baseline, not the target); `triton_reference` times the reference's Triton kernels
on the same GPU. `--impl reference` times only the CPU path, as the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, L, D_MODEL = 8, 2048, 1024
C = D_MODEL // 2
BYTES_PER_TOKEN_FWD = (3 * C + 4 * C) * 4           # read raw, write read
BYTES_PER_TOKEN_BWD = (3 * C + 4 * C + 3 * C) * 4   # read raw + grad_read, write grad_raw
BYTES_PER_TOKEN = BYTES_PER_TOKEN_FWD + BYTES_PER_TOKEN_BWD
FP32_TOL, BF16_TOL = 1e-5, 2e-2
KERNEL_LAUNCHES_PER_STEP = 5   # forward: fill + kernel; backward: fill + kernel + parameter-gradient reduce
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per step from the ncu capture of this workload
# (forward 102.2 + 134.2 MB, backward 323.3 + 100.7 MB; writes still in L2 at kernel end counted in full)
NCU_DRAM_BYTES_PER_STEP = 660.4e6
LONG_L = 65536


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def init_parameters(device):
    """lambda and gamma of a freshly initialised mixer (reference :1156-1173)."""
    ring = torch.linspace(0.85, 0.999, C)
    theta = torch.linspace(0.03, torch.pi * 0.97, C)
    tr, ti = ring * torch.cos(theta), ring * torch.sin(theta)
    gamma = torch.sqrt((1 - ring.square()).clamp_min(1e-4))
    return tr.to(device), ti.to(device), gamma.to(device)


def synthetic_inputs(seed: int, batch: int, length: int):
    """raw ~ N(0, 0.577^2) (what write_proj gives at init on N(0,1) input) and N(0,1) upstream
    gradients, rounded to bf16 and held in fp32 as autocast hands them to the operator."""
    gen = torch.Generator().manual_seed(seed)
    raw = (torch.randn(batch, length, 3 * C, generator=gen) * 0.577).bfloat16().float()
    grad_read = torch.randn(batch, length, 4 * C, generator=gen).bfloat16().float()
    return raw, grad_read


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---------------------------------------------------------------------------
# CPU side: the reference's own complex64 PyTorch path on the host cores
# ---------------------------------------------------------------------------
def cpu_reference():
    """(function, kind, description): the reference's `reference_field_read`
    (field_only_v4_chunked_triton_wiki100.py:392-416) from the staged copy, kind "reference";
    where that copy is absent, the pinned port of it, kind "port"."""
    from oracle import ref
    if ref.available():
        canon = ref.load_canon()
        return (lambda raw, tr, ti, gamma: canon.reference_field_read(raw, tr, ti, gamma, 32),
                "reference", "the reference's reference_field_read (complex64 hierarchical scan, "
                             "chunk 32) + PyTorch autograd, staged copy of the reference")
    from oracle import torch_port
    return (lambda raw, tr, ti, gamma: torch_port.field_read(raw, tr, ti, gamma, 32), "port",
            "complex64 PyTorch port of the reference's reference_field_read + autograd "
            f"({ref.why_unavailable()})")


def cpu_step(fn, raw, grad_read, tr, ti, gamma):
    """One forward + backward on the CPU; returns seconds."""
    raw = raw.clone().requires_grad_(True)
    tr, ti, gamma = (p.clone().requires_grad_(True) for p in (tr, ti, gamma))
    t0 = time.perf_counter()
    read = fn(raw, tr, ti, gamma)
    read.backward(grad_read)
    return time.perf_counter() - t0


def cpu_baseline(sample_batch: int = B, iters: int = 3):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fn, kind, what = cpu_reference()
    tr, ti, gamma = init_parameters("cpu")
    raw, grad_read = synthetic_inputs(1, sample_batch, L)
    cpu_step(fn, raw, grad_read, tr, ti, gamma)  # warm-up
    secs = [cpu_step(fn, raw, grad_read, tr, ti, gamma) for _ in range(iters)]
    return {"value": sample_batch * L / statistics.median(secs), "unit": "tokens/s",
            "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"forward+backward of {sample_batch} x {L} tokens (of the {B} x {L} "
                      f"workload), median of {iters} after 1 warm-up; {what}"}


def run_reference_arm(args, rank: int):
    """The reference's CPU implementation of the path, all host threads, bounded sample per step."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fn, kind, what = cpu_reference()
    tr, ti, gamma = init_parameters("cpu")
    raw, grad_read = synthetic_inputs(1, B, L)
    # bound the whole run to a few minutes: use fewer batch rows per step if the full batch is too slow
    t_full = cpu_step(fn, raw, grad_read, tr, ti, gamma)
    time_limit_s = 150.0
    sample_batch = B
    if (args.steps + args.warmup) * t_full > time_limit_s:
        sample_batch = max(1, min(B, int(B * time_limit_s / ((args.steps + args.warmup) * t_full))))
        raw, grad_read = raw[:sample_batch].contiguous(), grad_read[:sample_batch].contiguous()
    for _ in range(args.warmup):
        cpu_step(fn, raw, grad_read, tr, ti, gamma)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(fn, raw, grad_read, tr, ti, gamma)
    total = time.perf_counter() - t0
    value = sample_batch * L * args.steps / total
    sample = (f"each step = forward+backward of {sample_batch} x {L} tokens (of the {B} x {L} "
              f"workload); {what}")
    line = {
        "impl": "reference", "metric": "field_tokens_per_s_fwd_bwd", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(),
                         "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int):
    return {"workload": "field_block_recurrence_fwd_bwd_8x2048_d1024",
            "batch_per_gpu": B, "seq_len": L, "d_model": D_MODEL, "channels": C,
            "global_batch": B * n_gpus, "parallelism": f"batch-sharded x{n_gpus}, no collective",
            "boundary": "fused_field_read fp32 I/O (bf16-rounded activations), fp32 state",
            "cache": "inputs+outputs 448 MiB per step, larger than the 126 MB L2",
            "tolerances": {"fp32_rel": FP32_TOL, "bf16_rel_max_abs": BF16_TOL}}


# ---------------------------------------------------------------------------
# GPU side
# ---------------------------------------------------------------------------
def gpu_step(raw, grad_read, tr, ti, gamma):
    """One forward + backward through the public operator; returns (read, grad_raw)."""
    from fields_lm_b200 import fused_field_read
    raw.grad = tr.grad = ti.grad = gamma.grad = None
    read = fused_field_read(raw, tr, ti, gamma, 32, 64)
    read.backward(grad_read)
    return read, raw.grad


class DirectOp:
    """Forward and backward through the C ABI on preallocated buffers (what the autograd
    function does, minus the allocations): the device-resident hot path that `value` times."""

    def __init__(self, device, batch, length):
        from fields_lm_b200 import _lib
        self.lib = _lib.load()
        self.dims = (batch, length, C)
        self.read = torch.empty(batch, length, 4 * C, device=device)
        self.grad_raw = torch.empty(batch, length, 3 * C, device=device)
        self.grad_par = torch.empty(3, C, device=device)
        self.nf = self.lib.fields_read_workspace_bytes(batch, length, C, 0)
        self.nb = self.lib.fields_read_workspace_bytes(batch, length, C, 1)
        self.wsf = torch.empty(max(self.nf, 256), dtype=torch.uint8, device=device)
        self.wsb = torch.empty(max(self.nb, 256), dtype=torch.uint8, device=device)
        self.stream = torch.cuda.current_stream(device).cuda_stream

    def forward(self, raw, tr, ti, gamma):
        rc = self.lib.fields_read_forward(raw.data_ptr(), tr.data_ptr(), ti.data_ptr(),
                                          gamma.data_ptr(), None, self.read.data_ptr(), None,
                                          self.wsf.data_ptr(), self.nf, *self.dims, self.stream)
        if rc:
            raise RuntimeError(f"fields_read_forward status {rc}")

    def backward(self, raw, tr, ti, gamma, grad_read):
        g = self.grad_par
        rc = self.lib.fields_read_backward(raw.data_ptr(), tr.data_ptr(), ti.data_ptr(),
                                           gamma.data_ptr(), None, self.read.data_ptr(),
                                           grad_read.data_ptr(), None, self.grad_raw.data_ptr(),
                                           g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), None,
                                           self.wsb.data_ptr(), self.nb, *self.dims, self.stream)
        if rc:
            raise RuntimeError(f"fields_read_backward status {rc}")

    def status(self):
        """Error word of the last forward (single-pass kernels only write it)."""
        return self.lib.fields_read_device_status(self.wsf.data_ptr(), self.stream)


def bf16_leg(device, raw, grad_read, tr, ti, gamma, steps, stream):
    """Forward + backward through fields_read_*_bf16 on preallocated buffers (17,408 B/token)."""
    from fields_lm_b200 import _lib
    lib = _lib.load()
    raw16, grad16 = raw.bfloat16(), grad_read.bfloat16()
    read16 = torch.empty(B, L, 4 * C, device=device, dtype=torch.bfloat16)
    graw16 = torch.empty(B, L, 3 * C, device=device, dtype=torch.bfloat16)
    gpar = torch.empty(3, C, device=device)
    nf = lib.fields_read_workspace_bytes(B, L, C, 0)
    nb = lib.fields_read_workspace_bytes(B, L, C, 1)
    ws = torch.empty(max(nf, nb, 256), dtype=torch.uint8, device=device)
    st = stream.cuda_stream

    def step():
        rc = lib.fields_read_forward_bf16(raw16.data_ptr(), tr.data_ptr(), ti.data_ptr(),
                                          gamma.data_ptr(), None, read16.data_ptr(), None,
                                          ws.data_ptr(), nf, B, L, C, st)
        rc = rc or lib.fields_read_backward_bf16(
            raw16.data_ptr(), tr.data_ptr(), ti.data_ptr(), gamma.data_ptr(), None,
            read16.data_ptr(), grad16.data_ptr(), None, graw16.data_ptr(), gpar[0].data_ptr(),
            gpar[1].data_ptr(), gpar[2].data_ptr(), None, ws.data_ptr(), nb, B, L, C, st)
        if rc:
            raise RuntimeError(f"bf16 step status {rc}")
    for _ in range(3):
        step()
    ms = timed_loop(step, steps, stream) / steps
    return {"workload": "same step with bfloat16 raw/read/grad_read/grad_raw, fp32 state",
            "ms_per_step": ms, "algorithmic_bytes_per_token": BYTES_PER_TOKEN // 2}


DECODE_BATCH, DECODE_BLOCKS = 256, 18
DECODE_BYTES_PER_SEQ_BLOCK = 2 * (2 * C * 4) + 3 * C * 2 + 4 * C * 2   # state r+w, bf16 raw, bf16 read


def reference_field_block(device):
    """The reference's own `FieldBlock(1024, "triton", 32, 32, 64, 2528)` from the staged copy,
    seed-0 weights, on the GPU, and the module it lives in."""
    from oracle import ref
    canon = ref.load_canon()
    torch.manual_seed(0)
    return canon, canon.FieldBlock(D_MODEL, "triton", 32, 32, 64, 2528).to(device).train()


def block_leg(device, stream, iters: int = 10):
    """Forward + backward of one whole Field block of the reference (mixer + SwiGLU, d_model
    1,024, 8 x 2,048 tokens, autocast bf16), three ways: with the reference's Triton kernels, with
    this library installed at the operator boundary, and with `install(fused_mixer=True)`
    (bfloat16 boundary, norm statistics from the recurrence kernel). The GEMMs, norms and the
    feed-forward are PyTorch library calls in all three."""
    import fields_lm_b200
    from oracle import ref
    if not ref.available():
        return {"unavailable": ref.why_unavailable()}
    canon, block = reference_field_block(device)
    gen = torch.Generator(device=device).manual_seed(5)
    x = torch.randn(B, L, D_MODEL, device=device, generator=gen)
    gy = torch.randn(B, L, D_MODEL, device=device, generator=gen)

    def step():
        block.zero_grad(set_to_none=True)
        xg = x.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = block(xg)
        y.backward(gy)
        return y, xg.grad

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))

    out = {"workload": f"one reference FieldBlock forward + backward, {B} x {L} tokens, d_model "
                       f"{D_MODEL}, autocast bf16, seed-0 weights"}
    base = None
    for name, mode in (("reference_triton_kernels", None), ("operator_installed", False),
                       ("fused_mixer_installed", True)):
        try:
            if mode is not None:
                fields_lm_b200.install(block, fused_mixer=mode)
            for _ in range(3):
                y, gx = step()
            torch.cuda.reset_peak_memory_stats(device)
            ms = timed_loop(step, iters, stream) / iters
            out[name] = {"ms": ms, "tokens_per_s": B * L / (ms * 1e-3),
                         "peak_mib": torch.cuda.max_memory_allocated(device) / 2 ** 20}
            if base is None:
                base = (y.detach().clone(), gx.clone())
            else:
                out[name]["rel_vs_triton"] = {"y": rel(y.detach(), base[0]), "grad_x": rel(gx, base[1]),
                                              "tolerance": BF16_TOL}
        except Exception as exc:
            out[name] = {"error": repr(exc)[:300]}
        finally:
            if mode is not None:
                fields_lm_b200.uninstall(block)
    del block, x, gy
    return out


def block_breakdown(device, iters: int = 5):
    """Kernel-time table of the reference mixer's forward + backward with
    `install(fused_mixer=True)` (torch profiler): where the time of a Field block goes around the
    operator. Not part of the JSON line."""
    import fields_lm_b200
    from torch.profiler import ProfilerActivity, profile
    canon, block = reference_field_block(device)
    fields_lm_b200.install(block, fused_mixer=True)
    gen = torch.Generator(device=device).manual_seed(5)
    x = torch.randn(B, L, D_MODEL, device=device, generator=gen)
    gy = torch.randn(B, L, D_MODEL, device=device, generator=gen)

    def step():
        block.zero_grad(set_to_none=True)
        xg = x.requires_grad_(True)
        xg.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = block.mixer(xg)
        y.backward(gy)

    for _ in range(3):
        step()
    torch.cuda.synchronize(device)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(iters):
            step()
        torch.cuda.synchronize(device)
    print(f"mixer forward + backward, {B} x {L} tokens, d_model {D_MODEL}, {iters} iterations")
    print(prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=24,
                                    max_name_column_width=64))


def triton_reference_leg(device, stream, raw, grad_read, tr, ti, gamma, steps, ours_read,
                         ours_grad_raw):
    """The comparator this library displaces: the reference's six Triton kernels behind
    `fused_field_read` (field_only_v4_chunked_triton_wiki100.py:443-1123, geometry BLOCK_C 32 /
    CHUNK_T 64), JIT-compiled for this GPU, timed with CUDA events on the same tensors: forward
    + backward of 8 x 2,048 through its autograd function (as its callers run it), the same
    through this library's autograd function, and the forward of 1 x 65,536."""
    from oracle import ref
    from fields_lm_b200 import fused_field_read as ours
    if not ref.available():
        return {"unavailable": ref.why_unavailable()}
    peak = measured_peaks()[0]
    try:
        canon = ref.load_canon()
        theirs = canon.fused_field_read
        raw_g = raw.detach().clone().requires_grad_(True)
        par = [p.detach().clone().requires_grad_(True) for p in (tr, ti, gamma)]
        box = {}

        def make_step(fn):
            def step():
                raw_g.grad = None
                for q in par:
                    q.grad = None
                read = fn(raw_g, *par, 32, 64)
                read.backward(grad_read)
                box["read"] = read
            return step

        def rel(a, b):
            return float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))

        out = {"what": "reference Triton kernels (BLOCK_C 32, CHUNK_T 64) on this GPU, through the "
                       "reference's autograd function; `ours_autograd_ms` is this library through "
                       "its autograd function on the same tensors"}
        timings = {}
        for name, fn in (("triton", theirs), ("ours", ours)):
            step = make_step(fn)
            for _ in range(3):
                step()
            timings[name] = timed_loop(step, steps, stream) / steps
            if name == "triton":
                out["parity_vs_triton"] = {
                    "read_rel": rel(ours_read, box["read"].detach()),
                    "grad_raw_rel": rel(ours_grad_raw, raw_g.grad), "tolerance": FP32_TOL}
        ms = timings["triton"]
        out["fwd_bwd_8x2048"] = {
            "ms": ms, "tokens_per_s": B * L / (ms * 1e-3),
            "achieved": B * L * BYTES_PER_TOKEN / (ms * 1e-3) / 1e9,
            "frac": B * L * BYTES_PER_TOKEN / (ms * 1e-3) / 1e9 / peak,
            "ours_autograd_ms": timings["ours"]}
        box.clear()
        raw_g.grad = None
        long_raw = synthetic_inputs(2, 1, LONG_L)[0].to(device)
        tr_d, ti_d, gm_d = tr.detach(), ti.detach(), gamma.detach()

        def long_fwd():
            with torch.no_grad():
                theirs(long_raw, tr_d, ti_d, gm_d, 32, 64)
        for _ in range(3):
            long_fwd()
        n = max(5, min(steps, 30))
        ms = timed_loop(long_fwd, n, stream) / n
        out["fwd_1x65536"] = {
            "ms": ms, "tokens_per_s": LONG_L / (ms * 1e-3),
            "achieved": LONG_L * BYTES_PER_TOKEN_FWD / (ms * 1e-3) / 1e9,
            "frac": LONG_L * BYTES_PER_TOKEN_FWD / (ms * 1e-3) / 1e9 / peak}
        del long_raw
        return out
    except Exception as exc:  # Triton could not compile or run here: say why, keep the line
        return {"unavailable": f"reference Triton path failed on this box: {exc!r}"[:600]}


def real_scan_leg(device, stream, steps: int):
    """The softpatch mixer's scan at its size in the full model (8 x 2,048 tokens, rank 64, one
    decay per token expanded over the channels), forward + backward through autograd: the
    reference's `hierarchical_scan` (PyTorch ops on this GPU) and `fields_lm_b200.linear_scan`."""
    import fields_lm_b200
    from oracle import ref
    if not ref.available():
        return {"unavailable": ref.why_unavailable()}
    canon = ref.load_canon()
    gen = torch.Generator().manual_seed(5)
    rank = 64
    boundary0 = torch.rand(B, L, generator=gen).clamp(0.01, 0.99).to(device)
    z0 = torch.randn(B, L, rank, generator=gen).to(device)
    g = torch.randn(B, L, rank, generator=gen).to(device)
    out = {"workload": f"hierarchical_scan(a, drive, block=32) forward + backward, a = 1 - boundary "
                       f"expanded over {rank} channels, {B} x {L} tokens, fp32, through autograd"}
    results = {}
    for name, fn in (("reference_pytorch_ops", canon.hierarchical_scan),
                     ("this_library", fields_lm_b200.linear_scan)):
        boundary = boundary0.clone().requires_grad_(True)
        z = z0.clone().requires_grad_(True)

        def step():
            boundary.grad = z.grad = None
            a = (1.0 - boundary)[..., None].expand_as(z)
            state = fn(a, boundary[..., None] * z, block=32)
            state.backward(g)
            return state
        for _ in range(3):
            step()
        n = max(10, min(steps, 50))
        out[name] = {"ms": timed_loop(step, n, stream) / n}
        state = step()
        results[name] = [state.detach(), boundary.grad.clone(), z.grad.clone()]
    rel = [float((a - b).abs().max() / b.abs().max())
           for a, b in zip(results["this_library"], results["reference_pytorch_ops"])]
    out["parity_vs_reference"] = {"state_rel": rel[0], "grad_boundary_rel": rel[1],
                                  "grad_z_rel": rel[2], "tolerance": FP32_TOL}
    out["speedup"] = out["reference_pytorch_ops"]["ms"] / out["this_library"]["ms"]
    return out


def block_64k_leg(device, stream, dist_on: bool, rank: int, world: int, iters: int = 10):
    """Block-level strong scaling: the forward of ONE of the reference's Field blocks (staged
    copy, seed-0 weights, d_model 1,024, bf16 autocast, no_grad) over 1 x 65,536 tokens. On one
    GPU the whole sequence with the operator installed; on N GPUs every rank runs its span of the
    tokens through the same block and only the operator communicates (the one-launch sharded
    forward, summaries over NVLink peer stores); the projections, norms, gate and SwiGLU are
    token-parallel. The gathered output is compared with rank 0's single-GPU pass."""
    import fields_lm_b200
    from oracle import ref
    if not ref.available():
        return {"unavailable": ref.why_unavailable()}
    from fields_lm_b200 import seqpar
    canon, block = reference_field_block(device)
    block.eval()
    gen = torch.Generator().manual_seed(2)
    x_full = torch.randn(1, LONG_L, D_MODEL, generator=gen)
    lo, hi = seqpar.span_bounds(LONG_L, world, rank) if dist_on else (0, LONG_L)
    x = x_full[:, lo:hi].contiguous().to(device)
    sp = seqpar.SequenceParallelForwardFused(1, hi - lo, C, device) if dist_on else None

    def sharded_read(raw, tr, ti, gamma, block_c=None, chunk_t=None):
        read, _ = sp(raw.contiguous(), tr.contiguous(), ti.contiguous(), gamma.contiguous())
        return read

    fields_lm_b200.install(block, sharded_read if dist_on else fields_lm_b200.fused_field_read)

    def run():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            return block(x)
    try:
        for _ in range(3):
            run()
        barrier(dist_on)
        ms = max_over_ranks(timed_loop(run, iters, stream) / iters, dist_on, device)
        barrier(dist_on)
        y = run().float()
        status = sp.status() if sp is not None else 0
    finally:
        fields_lm_b200.uninstall(block)
    out = {"workload": "forward of one reference FieldBlock (mixer + SwiGLU, d_model 1,024) over "
                       f"1 x {LONG_L} tokens, bf16 autocast, no_grad" +
                       (f", tokens sharded over {world} GPUs, operator through "
                        "fields_read_forward_sharded" if dist_on else " on one GPU"),
           "scaling": "strong", "n_gpus": world, "ms": ms, "tokens_per_s": LONG_L / (ms * 1e-3),
           "status": status, "parity": None}
    if dist_on:
        parts = [torch.empty_like(y) for _ in range(world)] if rank == 0 else None
        # spans have equal length here (65,536 divides by the world sizes of one node)
        torch.distributed.gather(y, parts, dst=0)
        if rank == 0:
            del sp
            fields_lm_b200.install(block)
            try:
                with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                    want = block(x_full.to(device)).float()
            finally:
                fields_lm_b200.uninstall(block)
            got = torch.cat(parts, dim=1)
            out["parity"] = {"y_rel_vs_single_gpu": float((got - want).abs().max() / want.abs().max()),
                             "tolerance": BF16_TOL, "ranks": world}
    return out


def recurrence_kernel_share(step, device):
    """Share of one step's GPU kernel time spent in Field-recurrence kernels (torch profiler)."""
    from torch.profiler import ProfilerActivity, profile
    torch.cuda.synchronize(device)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize(device)
    total = field = 0.0
    for ev in prof.key_averages():
        t = float(getattr(ev, "self_device_time_total", 0.0) or 0.0)
        total += t
        key = ev.key
        if ("_field_" in key or "fields::" in key or "fill_entry" in key):
            field += t
    return field / total if total > 0 else None


def full_model_leg(device, stream, iters: int = 3):
    """One training step of the reference's full 24-layer model (18 Field / 2 Mamba-2 / 4 refresh
    blocks + PCAF, about 300 M parameters, seed 0) on token ids uniform in [0, 16384) of shape
    [8, 2048] under bf16 autocast, through the reference's public API: once with the reference's
    Triton Field kernels, once with this library installed; same model object, same weights."""
    import fields_lm_b200
    from oracle import full_model, mamba_standin, ref
    if not ref.available():
        return {"unavailable": ref.why_unavailable()}
    try:
        model, standin = full_model.build(device, model_seed=0)
        model.train()
        ids, labels = full_model.token_batch(B, L, 11, device)

        def step():
            return full_model.training_step(model, ids, labels)

        out = {"workload": f"FieldsForCausalLM(ids [{B}, {L}], labels) forward + backward, bf16 "
                           "autocast, fp32 weights from model_seed 0, checkpoint policy field_half",
               "parameters": sum(q.numel() for q in model.parameters()),
               "field_blocks": full_model.field_block_count(model),
               "mamba2": mamba_standin.STANDIN_LABEL if standin else "mamba-ssm package"}
        runs = {}
        for name in ("reference_triton_kernels", "operator_installed"):
            if name == "operator_installed":
                fields_lm_b200.install(model, scan=True)   # Field read + the softpatch mixer's scan
            for _ in range(2):
                step()
            ms = timed_loop(step, iters, stream) / iters
            loss = float(step())
            runs[name] = (loss, full_model.gradients(model), full_model.reads_by_block(model, ids))
            out[name] = {"ms": ms, "tokens_per_s": B * L / (ms * 1e-3), "loss": loss,
                         "recurrence_kernel_share": recurrence_kernel_share(step, device)}
            if name == "reference_triton_kernels":
                # The floor under the comparison: the reference against itself with its other
                # chunk length (32 steps instead of 64), which perturbs `read` at fp32 rounding level.
                full_model.set_triton_geometry(model, 32, 32)
                alt_loss = float(step())
                alt = (full_model.gradients(model), full_model.reads_by_block(model, ids))
                full_model.set_triton_geometry(model, 32, 64)
        fields_lm_b200.uninstall(model)
        want = runs["reference_triton_kernels"]

        def read_errors(reads):
            return [float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))
                    for a, b in zip(reads, want[2])]

        def grad_figures(grads):
            worst, where = full_model.compare_gradients(grads, want[1])
            wnorm, where_norm = full_model.norm_relative(grads, want[1])
            return {"grad_rel_worst": worst, "grad_worst_parameter": where,
                    "grad_norm_rel_worst": wnorm, "grad_norm_worst_parameter": where_norm}

        ours = runs["operator_installed"]
        out["parity"] = {
            "loss_abs": abs(ours[0] - want[0]), **grad_figures(ours[1]),
            "read_rel_by_field_block": read_errors(ours[2]),
            "tolerance": BF16_TOL,
            "floor_reference_vs_itself_chunk_32": {
                "loss_abs": abs(alt_loss - want[0]), **grad_figures(alt[0]),
                "read_rel_by_field_block": read_errors(alt[1])},
            "note": "the first Field block sees identical inputs on both sides (operator parity in "
                    "situ); later blocks see what 24 bf16 layers make of an fp32-rounding-level "
                    "difference, which the floor measures on the reference alone"}
        out["speedup"] = out["reference_triton_kernels"]["ms"] / out["operator_installed"]["ms"]
        del alt
        del model, runs
        torch.cuda.empty_cache()
        return out
    except Exception as exc:
        return {"unavailable": f"full model step failed: {exc!r}"[:600]}


def decode_leg(device, tr, ti, gamma, peak_gbs: float, iters: int = 200):
    from fields_lm_b200 import _lib
    lib = _lib.load()
    gen = torch.Generator().manual_seed(3)
    raws = [torch.randn(DECODE_BATCH, 3 * C, generator=gen).to(device).bfloat16()
            for _ in range(DECODE_BLOCKS)]
    states = [torch.randn(DECODE_BATCH, 2 * C, generator=gen).to(device) for _ in range(DECODE_BLOCKS)]
    reads = [torch.empty(DECODE_BATCH, 4 * C, device=device, dtype=torch.bfloat16)
             for _ in range(DECODE_BLOCKS)]

    def token_step():
        st = torch.cuda.current_stream(device).cuda_stream
        for raw, state, read in zip(raws, states, reads):
            rc = lib.fields_read_step_bf16(raw.data_ptr(), tr.data_ptr(), ti.data_ptr(),
                                           gamma.data_ptr(), state.data_ptr(), read.data_ptr(),
                                           DECODE_BATCH, C, st)
            if rc:
                raise RuntimeError(f"fields_read_step_bf16 status {rc}")

    stream = torch.cuda.current_stream(device)
    for _ in range(5):
        token_step()
    ms_plain = timed_loop(token_step, iters, stream) / iters
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device)
    side.wait_stream(stream)
    with torch.cuda.stream(side):
        token_step()
    stream.wait_stream(side)
    with torch.cuda.graph(graph):
        token_step()
    for _ in range(5):
        graph.replay()
    ms_graph = timed_loop(graph.replay, iters, stream) / iters
    nbytes = DECODE_BATCH * DECODE_BLOCKS * DECODE_BYTES_PER_SEQ_BLOCK
    parity = decode_parity(device)

    def gbs(ms):
        return nbytes / (ms * 1e-3) / 1e9
    return {"workload": f"one token x {DECODE_BATCH} sequences x {DECODE_BLOCKS} Field recurrences, "
                        "bf16 rows, fp32 states",
            "bytes_per_token_step": nbytes,
            "plain": {"ms": ms_plain, "achieved": gbs(ms_plain), "frac": gbs(ms_plain) / peak_gbs},
            "cuda_graph": {"ms": ms_graph, "achieved": gbs(ms_graph), "frac": gbs(ms_graph) / peak_gbs},
            "parity": parity,
            "note": "3.9 MB per launch: launch-latency scale, far below what HBM could move"}


def decode_parity(device, steps: int = 4, checked: int = 2):
    """Decode at its stated size against the reference: ids -> embedding -> 18 reference Field
    blocks (d_model 1,024, seed 0), batch 256, prefix 2,048, then `steps` single-token steps with
    bf16 per-step inputs and fp32 carried states; the oracle is the reference's full-sequence
    CPU pass (backend "reference") over prefix + steps tokens for the first `checked` sequences."""
    from oracle import decode_stack, ref
    if not ref.available():
        return {"unavailable": ref.why_unavailable()}
    try:
        cpu, gpu = decode_stack.build_pair(device)
        prefix = 2048
        ids = decode_stack.token_ids(DECODE_BATCH, prefix + steps)
        want_out, want_states = decode_stack.reference_full_pass(cpu, ids[:checked])
        got, trail = decode_stack.prefill_then_steps(gpu, ids, prefix, autocast_steps=True)

        def rel(a, b):
            return float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))
        out = {"what": f"{DECODE_BLOCKS} reference Field blocks, batch {DECODE_BATCH}, prefix "
                       f"{prefix}, {steps} steps under bf16 autocast vs the reference's fp32 CPU "
                       f"full pass of the first {checked} sequences",
               "step_output_rel": rel(got[:checked].cpu(), want_out[:, prefix:]),
               "carried_state_rel": max(rel(st[:checked].cpu(), want_states[b][:, -1])
                                        for b, st in enumerate(trail[-1])),
               "tolerance": BF16_TOL}
        del cpu, gpu, trail, got
        torch.cuda.empty_cache()
        return out
    except Exception as exc:
        return {"unavailable": f"decode parity failed: {exc!r}"[:400]}


class SpanOps:
    """One rank's share of a sharded forward on ONE GPU, without peers (P = 1): the one-launch
    kernel, the plain forward of the same span, and the summary pass of the three-launch form."""

    def __init__(self, device, tokens, tr, ti, gamma):
        import ctypes
        from fields_lm_b200 import _lib
        self.lib, self.T = _lib.load(), tokens
        self.raw = synthetic_inputs(2, 1, tokens)[0].to(device)
        self.par = (tr, ti, gamma)
        self.read = torch.empty(1, tokens, 4 * C, device=device)
        self.read2 = torch.empty(1, tokens, 4 * C, device=device)
        self.state = torch.empty(1, 2 * C, device=device)
        self.summary = torch.empty(1, 4, C, device=device)
        self.mail = torch.zeros(self.lib.fields_read_mailbox_bytes(1, 1, C), dtype=torch.uint8,
                                device=device)
        self.peers = (ctypes.c_void_p * 1)(self.mail.data_ptr())
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.n0 = self.lib.fields_read_workspace_bytes(1, tokens, C, 0)
        self.ws = torch.empty(max(self.n0, 256), dtype=torch.uint8, device=device)
        self.st = torch.cuda.current_stream(device).cuda_stream
        self.epoch = 0

    def fused(self):
        self.epoch += 1
        tr, ti, gm = self.par
        rc = self.lib.fields_read_forward_sharded(
            self.raw.data_ptr(), tr.data_ptr(), ti.data_ptr(), gm.data_ptr(), None,
            self.read.data_ptr(), self.state.data_ptr(), None, self.peers, self.err.data_ptr(), 0, 1,
            self.epoch, 0, 1, self.T, C, self.st)
        if rc:
            raise RuntimeError(f"fields_read_forward_sharded status {rc}")

    def plain(self):
        tr, ti, gm = self.par
        rc = self.lib.fields_read_forward(self.raw.data_ptr(), tr.data_ptr(), ti.data_ptr(),
                                          gm.data_ptr(), None, self.read2.data_ptr(), None,
                                          self.ws.data_ptr(), self.n0, 1, self.T, C, self.st)
        if rc:
            raise RuntimeError(f"fields_read_forward status {rc}")

    def summary_pass(self):
        tr, ti, gm = self.par
        rc = self.lib.fields_read_span_summary(self.raw.data_ptr(), tr.data_ptr(), ti.data_ptr(),
                                               gm.data_ptr(), self.summary.data_ptr(),
                                               self.ws.data_ptr(), self.n0, 1, self.T, C, self.st)
        if rc:
            raise RuntimeError(f"fields_read_span_summary status {rc}")


def span_leg(device, stream, tr, ti, gamma, iters: int = 50):
    """Per-rank times of the sharded 64K forward at 8, 4 and 2 ranks, measured on one GPU without
    the exchange: what the one-launch kernel costs over the plain forward of the same span."""
    peak = measured_peaks()[0]
    out = {"what": "one rank's span on one GPU, no peers: `one_launch_ms` = "
                   "fields_read_forward_sharded (P = 1), `plain_forward_ms` = fields_read_forward "
                   "of the same span (no summary), `summary_pass_ms` = fields_read_span_summary"}
    for tokens in (8192, 16384, 32768):
        ops = SpanOps(device, tokens, tr, ti, gamma)
        row = {}
        for name, fn in (("one_launch_ms", ops.fused), ("plain_forward_ms", ops.plain),
                         ("summary_pass_ms", ops.summary_pass)):
            for _ in range(3):
                fn()
            row[name] = timed_loop(fn, iters, stream) / iters
        ops.fused()
        ops.plain()
        row["parity_rel"] = float((ops.read - ops.read2).abs().max() / ops.read2.abs().max())
        row["status"] = int(ops.err.item())
        row["one_launch_frac"] = tokens * BYTES_PER_TOKEN_FWD / (row["one_launch_ms"] * 1e-3) / 1e9 / peak
        out[f"{tokens}_tokens"] = row
        del ops
    return out


class TensorExperiment:
    """The tcgen05 restatement of the bfloat16 forward (an experiment, not the production path)
    beside the production bfloat16 forward kernel, on the training shape."""

    def __init__(self, device, tr, ti, gamma):
        from fields_lm_b200 import _lib
        self.lib = _lib.load()
        self.par = (tr, ti, gamma)
        self.raw16 = synthetic_inputs(1, B, L)[0].to(device).bfloat16()
        self.read_tc = torch.empty(B, L, 4 * C, device=device, dtype=torch.bfloat16)
        self.read_sp = torch.empty(B, L, 4 * C, device=device, dtype=torch.bfloat16)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.n = self.lib.fields_read_workspace_bytes(B, L, C, 0)
        self.ws = torch.empty(max(self.n, 256), dtype=torch.uint8, device=device)
        self.st = torch.cuda.current_stream(device).cuda_stream

    def tensor(self):
        tr, ti, gm = self.par
        rc = self.lib.fields_read_forward_bf16_tensor(
            self.raw16.data_ptr(), tr.data_ptr(), ti.data_ptr(), gm.data_ptr(), None,
            self.read_tc.data_ptr(), None, self.err.data_ptr(), B, L, C, self.st)
        if rc:
            raise RuntimeError(f"fields_read_forward_bf16_tensor status {rc}")

    def single_pass(self):
        tr, ti, gm = self.par
        rc = self.lib.fields_read_forward_bf16(
            self.raw16.data_ptr(), tr.data_ptr(), ti.data_ptr(), gm.data_ptr(), None,
            self.read_sp.data_ptr(), None, self.ws.data_ptr(), self.n, B, L, C, self.st)
        if rc:
            raise RuntimeError(f"fields_read_forward_bf16 status {rc}")


def tensor_leg(device, stream, tr, ti, gamma, iters: int = 50):
    """Times the tcgen05 experiment against the production bfloat16 forward (8 x 2,048 tokens)."""
    try:
        ex = TensorExperiment(device, tr, ti, gamma)
        out = {"what": "forward of 8 x 2,048 tokens on the bfloat16 boundary: the prefix-ratio "
                       "contraction on tcgen05 (experiment) beside the production single-pass kernel; "
                       "its 2 x 128 x 128 x 64 flop per 128-step tile and 32 channels are "
                       f"{2 * 128 * 128 * 64 * (L // 128) * B * (C // 32) / 1e9:.1f} GFLOP per call"}
        for name, fn in (("tcgen05_ms", ex.tensor), ("single_pass_ms", ex.single_pass)):
            for _ in range(3):
                fn()
            out[name] = timed_loop(fn, iters, stream) / iters
        out["status"] = int(ex.err.item())
        out["rel_vs_single_pass"] = float((ex.read_tc.float() - ex.read_sp.float()).abs().max() /
                                          ex.read_sp.float().abs().max())
        out["tolerance"] = BF16_TOL
        flop = 2 * 128 * 128 * 64 * (L // 128) * B * (C // 32)
        out["tensor_tflops_if_only_mma"] = flop / (out["tcgen05_ms"] * 1e-3) / 1e12
        return out
    except Exception as exc:
        return {"unavailable": repr(exc)[:300]}


def timed_loop(fn, steps: int, stream) -> float:
    """Milliseconds for `steps` calls of fn, CUDA events on the launching stream."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop)


def barrier(dist_on: bool):
    if dist_on:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, dist_on: bool, device) -> float:
    if not dist_on:
        return x
    t = torch.tensor([x], device=device, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def parity_check(device, tr, ti, gamma):
    """Small live check against the CPU oracle so the line carries its own parity figure."""
    from oracle import field_oracle
    raw, grad_read = synthetic_inputs(7, 2, 256)
    r = raw.to(device).requires_grad_(True)
    p = [x.clone().requires_grad_(True) for x in (tr, ti, gamma)]
    read, grad_raw = gpu_step(r, grad_read.to(device), *p)
    ref_read, _ = field_oracle.forward(raw.numpy(), tr.cpu().numpy(), ti.cpu().numpy(),
                                       gamma.cpu().numpy())
    ref_grad = field_oracle.backward(raw.numpy(), tr.cpu().numpy(), ti.cpu().numpy(),
                                     gamma.cpu().numpy(), grad_read.numpy())[0]

    def rel(a, b):
        return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-6))

    return {"read_rel": rel(read.detach().cpu().numpy().astype(np.float64), ref_read),
            "grad_raw_rel": rel(grad_raw.cpu().numpy().astype(np.float64), ref_grad),
            "tolerance": FP32_TOL}


def pin_to_gpu_numa_node(index: int):
    """Moves this process onto the CPUs NVML names as closest to GPU `index` (a process
    setting: nothing of the GPU changes). Returns what was done, for the JSON line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if not cpus:
            return {"pinned": False, "why": "NVML's ideal CPUs are outside this process's cpuset"}
        os.sched_setaffinity(0, cpus)
        return {"pinned": True, "cpus": len(cpus), "of": os.cpu_count()}
    except Exception as exc:
        return {"pinned": False, "why": repr(exc)[:200]}


def pcie_rates(device, stream, host_pinned, device_like):
    """Plain pinned copies of one input tensor each way and both ways at once: the rate the box's
    host link gives, which bounds the end-to-end figure."""
    dev = torch.empty_like(device_like)
    back = torch.empty_like(host_pinned)
    nbytes = host_pinned.numel() * host_pinned.element_size()
    side = torch.cuda.Stream(device)

    def h2d():
        dev.copy_(host_pinned, non_blocking=True)

    def d2h():
        back.copy_(device_like, non_blocking=True)

    def both():
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            back.copy_(device_like, non_blocking=True)
        dev.copy_(host_pinned, non_blocking=True)
        stream.wait_stream(side)
    out = {"bytes_each_way": nbytes}
    for name, fn in (("h2d", h2d), ("d2h", d2h), ("both_ways", both)):
        fn()
        torch.cuda.synchronize(device)
        ms = timed_loop(fn, 3, stream) / 3
        out[name + "_ms"] = ms
        out[name + "_gbs"] = nbytes * (2 if name == "both_ways" else 1) / (ms * 1e-3) / 1e9
    return out


def run_ours(args, rank: int, world: int, local_rank: int):
    from fields_lm_b200 import _lib, fused_field_read
    _lib.load()  # raises if the CUDA library is missing: there is no fallback
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (use --impl reference for the CPU arm)")
    dist_on = world > 1
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if dist_on:
        torch.distributed.init_process_group("nccl", device_id=device)
    stream = torch.cuda.current_stream(device)

    tr, ti, gamma = (p.requires_grad_(True) for p in init_parameters(device))
    raw_h, grad_h = synthetic_inputs(1 + rank, B, L)
    raw = raw_h.to(device).requires_grad_(True)
    grad_read = grad_h.to(device)

    op = DirectOp(device, B, L)
    raw_d, tr_d, ti_d, gm_d = raw.detach(), tr.detach(), ti.detach(), gamma.detach()

    def step():
        op.forward(raw_d, tr_d, ti_d, gm_d)
        op.backward(raw_d, tr_d, ti_d, gm_d, grad_read)
    for _ in range(max(args.warmup, 3)):
        step()
    if args.profile_bf16:
        # profiler capture of the step on the bfloat16 boundary, no JSON line
        bf16_leg(device, raw_d, grad_read, tr_d, ti_d, gm_d, args.steps, stream)
        torch.cuda.synchronize()
        print(f"profile run: {args.steps} bfloat16 steps done")
        return
    if args.profile_tensor:
        # profiler capture of the tcgen05 experiment beside the production bf16 forward
        ex = TensorExperiment(device, tr_d, ti_d, gm_d)
        for _ in range(2 + args.steps):
            ex.tensor()
            ex.single_pass()
        torch.cuda.synchronize()
        print(f"profile run: {args.steps} tensor-experiment and single-pass bf16 forwards, "
              f"status {int(ex.err.item())}")
        return
    if args.profile_span:
        # profiler capture of the one-launch sharded forward on one span, no peers, no JSON line
        ops = SpanOps(device, args.profile_span, tr_d, ti_d, gm_d)
        for _ in range(3 + args.steps):
            ops.fused()
        torch.cuda.synchronize()
        print(f"profile run: {args.steps} one-launch forwards of {args.profile_span} tokens, "
              f"status {int(ops.err.item())}")
        return
    if args.profile:
        # short path for profiler captures: a few plain steps, no host work, no JSON line
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
        print(f"profile run: {args.steps} steps done")
        return
    # The step's five launches (two workspace fills, forward, backward, reduction) are captured
    # once in a CUDA graph and replayed: the usual way to run a launch-bound step. The same steps
    # issued one by one are timed beside it (`plain_ms_per_step`).
    plain_step = step
    graph = None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device)
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                op.stream = side.cuda_stream
                plain_step()
            stream.wait_stream(side)
            with torch.cuda.graph(graph):
                op.stream = torch.cuda.current_stream(device).cuda_stream
                plain_step()
            op.stream = stream.cuda_stream
            step = graph.replay
            for _ in range(3):
                step()
        except Exception as exc:  # capture unsupported: keep the plain launches
            print(f"cuda graph capture failed, timing plain launches: {exc!r}", file=sys.stderr)
            graph = None
            op.stream = stream.cuda_stream
            step = plain_step
    with ClockSampler(local_rank) as clocks:
        barrier(dist_on)
        ms = timed_loop(step, args.steps, stream)
        barrier(dist_on)
        # keep the same steps running long enough for NVML to see clocks under this load
        t_end = time.perf_counter() + 0.4
        while time.perf_counter() < t_end:
            step()
            torch.cuda.synchronize()
    ms = max_over_ranks(ms, dist_on, device)
    ms_per_step = ms / args.steps
    ms_plain = timed_loop(plain_step, args.steps, stream) / args.steps
    tokens_per_s = world * B * L / (ms_per_step * 1e-3)

    # forward-only and backward-only, to split the step for the roofline report
    def fwd_only():
        op.forward(raw_d, tr_d, ti_d, gm_d)
    for _ in range(3):
        fwd_only()
    ms_fwd = timed_loop(fwd_only, args.steps, stream) / args.steps

    # secondary workload of the metric: forward of one 65,536-token sequence, on one GPU or
    # sharded over the sequence across all ranks (span summaries exchanged with NCCL)
    long_steps = max(5, min(args.steps, 50))
    if dist_on:
        from fields_lm_b200 import seqpar
        lo, hi = seqpar.span_bounds(LONG_L, world, rank)
        long_raw = synthetic_inputs(2, 1, LONG_L)[0][:, lo:hi].contiguous().to(device)
        # summaries through peer memory (NVLink stores); NCCL all_gather if symmetric memory is
        # unavailable or a warm-up exchange reports a timeout. The ranks decide together.
        def all_agree(ok: bool) -> bool:
            flag = torch.tensor([1 if ok else 0], device=device, dtype=torch.int32)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
            return bool(flag.item())
        # Preferred: the whole sharded forward as one cooperative launch per rank (summary sweep,
        # exchange over NVLink peer stores, fold and forward; the span read from HBM once). Then
        # the three-launch form over the same mailboxes, then NCCL all_gather. A form is used
        # only if every rank could build it and two warm-up calls report no timeout.
        sp_fwd, exchange, alternatives = None, None, {}
        long_call, best_ms = None, None

        def replayed(cand):
            """The call captured once in a CUDA graph (the kernel keeps its epoch on the device)."""
            cur = torch.cuda.current_stream(device)
            side = torch.cuda.Stream(device)
            side.wait_stream(cur)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                cand(long_raw, tr_d, ti_d, gm_d)
                with torch.cuda.graph(graph, stream=side):
                    cand(long_raw, tr_d, ti_d, gm_d)
            cur.wait_stream(side)
            torch.cuda.synchronize(device)

            def run():
                graph.replay()
                return cand.read, cand.state_out
            return run

        forms = (("one cooperative launch per rank, summaries over NVLink peer stores",
                  lambda: seqpar.SequenceParallelForwardFused(1, hi - lo, C, device), False),
                 ("the same launch replayed from a CUDA graph, epoch kept on the device",
                  lambda: seqpar.SequenceParallelForwardFused(1, hi - lo, C, device,
                                                              device_epoch=True), True),
                 ("three launches per rank, summaries over NVLink peer stores",
                  lambda: seqpar.SequenceParallelForwardP2P(1, hi - lo, C, device), False))
        for label, make, as_graph in forms:
            try:
                cand = make()
                built = True
            except Exception as exc:
                print(f"{label}: unavailable ({exc!r})", file=sys.stderr)
                cand, built = None, False
            healthy = False
            call = None
            if all_agree(built):
                for _ in range(3):
                    cand(long_raw, tr_d, ti_d, gm_d)
                healthy = all_agree(cand.status() == 0)
            if healthy and as_graph:
                try:
                    call = replayed(cand)
                except Exception as exc:
                    print(f"{label}: capture failed ({exc!r})", file=sys.stderr)
                    call = None
                healthy = all_agree(call is not None)
            elif healthy:
                call = (lambda c: (lambda: c(long_raw, tr_d, ti_d, gm_d)))(cand)
            if healthy:
                for _ in range(2):
                    call()
                barrier(dist_on)
                ms = max_over_ranks(timed_loop(call, long_steps, stream) / long_steps, dist_on, device)
                healthy = all_agree(cand.status() == 0)
            if healthy:
                alternatives[label] = ms
                if best_ms is None or ms < best_ms:
                    best_ms, sp_fwd, exchange, long_call = ms, cand, label, call
        healthy = sp_fwd is not None
        if not healthy:
            print("peer-memory exchange not usable here; using NCCL all_gather", file=sys.stderr)
            sp_fwd = seqpar.SequenceParallelForward(1, hi - lo, C, device)
            exchange = "three launches per rank, nccl all_gather"
            long_call = lambda: sp_fwd(long_raw, tr_d, ti_d, gm_d)
        long_fwd = long_call
    else:
        exchange, alternatives = None, None
        long_op = DirectOp(device, 1, LONG_L)
        long_raw = synthetic_inputs(2, 1, LONG_L)[0].to(device)
        long_fwd = lambda: long_op.forward(long_raw, tr_d, ti_d, gm_d)
    for _ in range(3):
        long_fwd()
    barrier(dist_on)
    ms_long = max_over_ranks(timed_loop(long_fwd, long_steps, stream) / long_steps, dist_on, device)
    barrier(dist_on)

    # Sharded runs prove their output, outside the timed region: every rank also runs the whole
    # sequence on its own GPU (the single-GPU path that the parity tests hold to the oracle) and
    # compares its span of `read` with that slice; the worst rank's figure goes into the line.
    long_parity = None
    full_long = None
    if dist_on:
        full_long = {"raw": synthetic_inputs(2, 1, LONG_L)[0].to(device)}
        full_op = DirectOp(device, 1, LONG_L)
        full_op.forward(full_long["raw"], tr_d, ti_d, gm_d)
        span_read, _ = long_fwd()
        want = full_op.read[:, lo:hi]
        err = float((span_read - want).abs().max() / full_op.read.abs().max().clamp_min(1e-6))
        long_parity = {"read_rel_vs_single_gpu": max_over_ranks(err, dist_on, device),
                       "tolerance": FP32_TOL, "ranks": world}
        full_long["op"] = full_op

    # the training step of the same sequence: forward + backward, on one GPU through the C ABI on
    # preallocated buffers, on several sharded over the sequence through the autograd function
    # (dual summaries all-gathered in the backward pass, parameter gradients all-reduced)
    full_grad = torch.randn(1, LONG_L, 4 * C, device=device,
                            generator=torch.Generator(device=device).manual_seed(3))
    long_grad = full_grad[:, lo:hi].contiguous() if dist_on else full_grad
    if dist_on:
        del sp_fwd  # its buffers; the training step holds its own
        if healthy:
            trainer = seqpar.SequenceParallelTrainStepP2P(1, hi - lo, C, device)
            train_api = ("seqpar.SequenceParallelTrainStepP2P (summaries and the parameter-gradient "
                         "sum over NVLink peer stores, no collective library in the step)")
        else:
            trainer = seqpar.SequenceParallelTrainStep(1, hi - lo, C, device)
            train_api = "seqpar.SequenceParallelTrainStep (NCCL all_gather x2, all_reduce)"

        def long_train():
            trainer.forward(long_raw, tr_d, ti_d, gm_d)
            trainer.backward(long_raw, tr_d, ti_d, gm_d, long_grad)
    else:
        def long_train():
            long_op.forward(long_raw, tr_d, ti_d, gm_d)
            long_op.backward(long_raw, tr_d, ti_d, gm_d, long_grad)
        train_api = "fields_read_forward + fields_read_backward on preallocated buffers"
    try:
        for _ in range(3):
            long_train()
        barrier(dist_on)
        train_steps = max(5, min(args.steps, 20))
        ms_train = max_over_ranks(timed_loop(long_train, train_steps, stream) / train_steps, dist_on,
                                  device)
        barrier(dist_on)
    except Exception as exc:  # the headline line must still be printed
        print(f"train_64k leg failed: {exc!r}", file=sys.stderr)
        ms_train = None
    # the same step with the parameter-gradient sum through one NCCL all_reduce, for comparison
    ms_train_nccl = None
    if dist_on and healthy and ms_train is not None:
        try:
            other = seqpar.SequenceParallelTrainStepP2P(1, hi - lo, C, device, nccl_reduce=True)

            def other_train():
                other.forward(long_raw, tr_d, ti_d, gm_d)
                other.backward(long_raw, tr_d, ti_d, gm_d, long_grad)
            for _ in range(3):
                other_train()
            barrier(dist_on)
            ms_train_nccl = max_over_ranks(timed_loop(other_train, train_steps, stream) / train_steps,
                                           dist_on, device)
            barrier(dist_on)
            del other
        except Exception as exc:
            print(f"train_64k NCCL-reduce comparison failed: {exc!r}", file=sys.stderr)
    train_parity = None
    if dist_on and ms_train is not None:
        full_op = full_long["op"]
        full_op.backward(full_long["raw"], tr_d, ti_d, gm_d, full_grad)
        trainer.forward(long_raw, tr_d, ti_d, gm_d)
        span_graw, span_gpar = trainer.backward(long_raw, tr_d, ti_d, gm_d, long_grad)
        want = full_op.grad_raw[:, lo:hi]
        e1 = float((span_graw - want).abs().max() / full_op.grad_raw.abs().max().clamp_min(1e-6))
        e2 = float((span_gpar - full_op.grad_par).abs().max() /
                   full_op.grad_par.abs().max().clamp_min(1e-6))
        train_parity = {"grad_raw_rel_vs_single_gpu": max_over_ranks(e1, dist_on, device),
                        "grad_params_rel_vs_single_gpu": max_over_ranks(e2, dist_on, device),
                        "tolerance": FP32_TOL, "ranks": world}
    del long_raw, long_grad, full_grad, full_long

    # the same step on the bfloat16 boundary (raw, read and their gradients in bf16, fp32 state)
    bf16 = bf16_leg(device, raw_d, grad_read, tr_d, ti_d, gm_d, args.steps, stream)

    # decode: one token for 256 sequences through the recurrences of 18 Field
    # blocks, bf16 rows, fp32 carried states; plain launches and one CUDA graph of the 18 launches
    decode = decode_leg(device, tr_d, ti_d, gm_d, peak_gbs=measured_peaks()[0]) if not dist_on else None
    block = block_leg(device, stream) if not dist_on else None
    spans = span_leg(device, stream, tr_d, ti_d, gm_d) if not dist_on else None
    tensor = tensor_leg(device, stream, tr_d, ti_d, gm_d) if not dist_on else None
    real_scan = real_scan_leg(device, stream, args.steps) if not dist_on else None
    # the reference's Triton kernels on this GPU, same tensors (rank 0's GPU only)
    triton = None
    if rank == 0 and not args.no_triton:
        read0, graw0 = gpu_step(raw, grad_read, tr, ti, gamma)
        triton = triton_reference_leg(device, stream, raw, grad_read, tr, ti, gamma,
                                      max(5, min(args.steps, 30)), read0.detach(), graw0)
        del read0, graw0
    full_model = full_model_leg(device, stream) if (not dist_on and not args.no_full_model) else None
    block_64k = None
    if not args.no_triton:   # needs the staged reference, like the Triton leg
        try:
            block_64k = block_64k_leg(device, stream, dist_on, rank, world)
        except Exception as exc:
            block_64k = {"unavailable": repr(exc)[:400]}

    # end to end: pinned host -> device, forward + backward, results back to pinned host.
    # The process first moves onto the CPUs next to its GPU (NVML's ideal affinity for the device),
    # so that the pinned buffers it allocates from here on sit on that NUMA node.
    all_cpus = os.sched_getaffinity(0)
    placement = pin_to_gpu_numa_node(local_rank)
    raw_pin, grad_pin = raw_h.pin_memory(), grad_h.pin_memory()
    read_pin = torch.empty(B, L, 4 * C).pin_memory()
    graw_pin = torch.empty(B, L, 3 * C).pin_memory()
    gpar_pin = torch.empty(3, C).pin_memory()

    from fields_lm_b200.host import HostFieldRead
    pipe = HostFieldRead(device, B, L, C, rows_per_chunk=1)

    # Steps are issued back to back, as a training loop with a prefetching loader does: every
    # step uploads its inputs and downloads its results, the next step's upload may run while the
    # previous step's download is still in flight, and the timed region ends when the last
    # result has reached the host.
    def e2e_steps_then_join(n):
        for _ in range(n):
            pipe.fwd_bwd(raw_pin, grad_pin, tr_d, ti_d, gm_d, read_pin, graw_pin, gpar_host=gpar_pin,
                         wait=False)
        pipe.join()
    e2e_steps_then_join(2)
    torch.cuda.synchronize(device)
    pcie = pcie_rates(device, stream, raw_pin, raw_d)
    e2e_steps = max(3, min(args.steps, 10))
    barrier(dist_on)
    ms_e2e = max_over_ranks(timed_loop(lambda: e2e_steps_then_join(e2e_steps), 1, stream) / e2e_steps,
                            dist_on, device)
    barrier(dist_on)
    os.sched_setaffinity(0, all_cpus)  # the CPU baseline below uses every host core again

    if rank != 0:
        if dist_on:
            torch.distributed.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    achieved = B * L * BYTES_PER_TOKEN / (ms_per_step * 1e-3) / 1e9 if world == 1 else \
        B * L * BYTES_PER_TOKEN / (ms_per_step * 1e-3) / 1e9
    fwd_gbs = B * L * BYTES_PER_TOKEN_FWD / (ms_fwd * 1e-3) / 1e9
    bwd_ms = max(ms_plain - ms_fwd, 1e-6)  # both halves from plain launches
    line = {
        "metric": "field_tokens_per_s_fwd_bwd", "value": tokens_per_s, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "plain_ms_per_step": ms_plain,
        "launch": "cuda graph replay of the step" if graph is not None else "plain launches",
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(world),
        "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "traffic": NCU_DRAM_BYTES_PER_STEP,
            "traffic_source": "ncu dram__bytes_read+write of the two single-pass kernels, "
                              "profiles/single_pass_fwd_bwd_8x2048_ncu.md",
            "peak_source": f"of {peak_kind}",
            "frac_of_nominal_8_tb_s": achieved / 8000.0,
            "kernel": "whole step per GPU: fill + FwdSinglePass + fill + BwdSinglePass + BwdReduce, dependent launches",
            "algorithmic_bytes_per_token": BYTES_PER_TOKEN,
            "forward": {"ms": ms_fwd, "achieved": fwd_gbs, "frac": fwd_gbs / peak},
            "backward": {"ms": bwd_ms,
                         "achieved": B * L * BYTES_PER_TOKEN_BWD / (bwd_ms * 1e-3) / 1e9,
                         "frac": B * L * BYTES_PER_TOKEN_BWD / (bwd_ms * 1e-3) / 1e9 / peak},
        },
        "e2e": {"value": world * B * L / (ms_e2e * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": raw_pin.numel() * 4 + grad_pin.numel() * 4,
                "d2h_bytes_per_step": (read_pin.numel() + graw_pin.numel() + gpar_pin.numel()) * 4,
                "ms_per_step": ms_e2e,
                "api": "fields_lm_b200.host.HostFieldRead.fwd_bwd: pinned host in/out, one batch "
                       "row per chunk, uploads / kernels / downloads overlapped on three streams "
                       "(read leaves after the forward while grad_read still arrives; steps issued "
                       "back to back, the timed region ends when the last result is on the host)",
                "host_placement": placement, "pcie": pcie,
                "bound": "PCIe: every step moves h2d + d2h bytes through the host link; "
                         "pcie.both_ways_ms is what plain copies of the same bytes take"},
        "forward_64k": {"workload": "forward of 1 x 65,536 tokens" +
                                    (f", sequence-sharded over {world} GPUs" if dist_on else " on one GPU"),
                        "scaling": "strong", "n_gpus": world, "exchange": exchange,
                        "ms_by_form": alternatives,
                        "ms": ms_long, "tokens_per_s": LONG_L / (ms_long * 1e-3),
                        "achieved": LONG_L * BYTES_PER_TOKEN_FWD / (ms_long * 1e-3) / 1e9,
                        "frac": LONG_L * BYTES_PER_TOKEN_FWD / (ms_long * 1e-3) / 1e9 / (peak * world),
                        "parity": long_parity},
        "train_64k": None if ms_train is None else {
            "workload": "forward + backward of 1 x 65,536 tokens" +
                        (f", sequence-sharded over {world} GPUs" if dist_on else " on one GPU"),
            "scaling": "strong", "n_gpus": world, "api": train_api, "ms": ms_train,
            "tokens_per_s": LONG_L / (ms_train * 1e-3),
            "achieved": LONG_L * BYTES_PER_TOKEN / (ms_train * 1e-3) / 1e9,
            "frac": LONG_L * BYTES_PER_TOKEN / (ms_train * 1e-3) / 1e9 / (peak * world),
            "ms_with_nccl_all_reduce_of_parameter_gradients": ms_train_nccl,
            "parity": train_parity},
        "bf16_io": {**bf16, "achieved": B * L * BYTES_PER_TOKEN / 2 / (bf16["ms_per_step"] * 1e-3) / 1e9,
                    "frac": B * L * BYTES_PER_TOKEN / 2 / (bf16["ms_per_step"] * 1e-3) / 1e9 / peak,
                    "tokens_per_s": world * B * L / (bf16["ms_per_step"] * 1e-3)},
        "decode_step": decode,
        "field_block": block,
        "field_block_64k": block_64k,
        "sharded_span_one_gpu": spans,
        "tcgen05_experiment": tensor,
        "real_scan": real_scan,
        "triton_reference": triton,
        "full_model": full_model,
        "gpu_launches": KERNEL_LAUNCHES_PER_STEP * args.steps,
        "clocks": clocks.summary(),
        "parity": parity_check(device, tr.detach(), ti.detach(), gamma.detach()),
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)
    if dist_on:
        torch.distributed.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true",
                    help="skip the CPU baseline leg (used for profiler runs)")
    ap.add_argument("--no-triton", action="store_true",
                    help="skip the leg that times the reference's Triton kernels on this GPU")
    ap.add_argument("--no-full-model", action="store_true",
                    help="skip the full 24-layer model leg")
    ap.add_argument("--no-graph", action="store_true",
                    help="time plain launches instead of a CUDA graph of the step")
    ap.add_argument("--block-breakdown", action="store_true",
                    help="print the kernel-time table of one fused mixer step and exit")
    ap.add_argument("--profile-bf16", action="store_true",
                    help="run only the forward + backward step on the bfloat16 boundary (for ncu)")
    ap.add_argument("--profile-tensor", action="store_true",
                    help="run only the tcgen05 experiment and the bf16 single-pass forward (for ncu)")
    ap.add_argument("--profile-span", type=int, default=0, metavar="TOKENS",
                    help="run only the one-launch sharded forward on a span of TOKENS (for ncu)")
    ap.add_argument("--profile", action="store_true",
                    help="run warm-up + steps only (for ncu captures); prints no bench line")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.block_breakdown:
        if not torch.cuda.is_available():
            raise SystemExit("--block-breakdown needs a CUDA device")
        torch.cuda.set_device(0)
        block_breakdown(torch.device("cuda", 0))
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
