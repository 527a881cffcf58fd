"""The forward entry point that allocates nothing, against the ordinary forward.

``fields_read_forward_noalloc`` serves hosts that cannot give the library a
workspace - an operator running inside an inference runtime's execution hook, a
plug-in of a serving engine with a memory plan fixed at start-up, a loop that must
not stall on cudaMalloc. It runs the same kernels as ``fields_read_forward`` on a
fixed 16 MiB buffer built into the library, so its output must equal the ordinary
entry point's. The buffer is shared by every call and keeps the previous call's
contents, so the check is made on two calls in a row with different inputs and
shapes. Collected last on purpose: a failure here stops nothing else.
"""
import numpy as np
import pytest
import torch

from conftest import FP32_TOL, rel_err

pytestmark = pytest.mark.gpu


def _inputs(dev, B, L, C, seed):
    gen = torch.Generator().manual_seed(seed)
    radius = torch.rand(C, generator=gen) * 0.49 + 0.5
    theta = (torch.rand(C, generator=gen) * 2 - 1) * torch.pi
    tr, ti = radius * torch.cos(theta), radius * torch.sin(theta)
    gamma = torch.sqrt((1 - radius.square()).clamp_min(1e-4))
    raw = torch.randn(B, L, 3 * C, generator=gen)
    state = torch.randn(B, 2 * C, generator=gen)
    return [t.to(dev).contiguous() for t in (raw, tr, ti, gamma, state)]


def _ordinary(lib, raw, tr, ti, gamma, state, B, L, C, stream):
    read = torch.empty(B, L, 4 * C, device=raw.device)
    out = torch.empty(B, 2 * C, device=raw.device)
    nbytes = lib.fields_read_workspace_bytes(B, L, C, 0)
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=raw.device)
    rc = lib.fields_read_forward(raw.data_ptr(), tr.data_ptr(), ti.data_ptr(), gamma.data_ptr(),
                                 state.data_ptr(), read.data_ptr(), out.data_ptr(), ws.data_ptr(),
                                 nbytes, B, L, C, stream)
    assert rc == 0
    return read, out


def _noalloc(lib, raw, tr, ti, gamma, state, B, L, C, stream):
    read = torch.full((B, L, 4 * C), float("nan"), device=raw.device)
    out = torch.full((B, 2 * C), float("nan"), device=raw.device)
    rc = lib.fields_read_forward_noalloc(raw.data_ptr(), tr.data_ptr(), ti.data_ptr(),
                                         gamma.data_ptr(), state.data_ptr(), read.data_ptr(),
                                         out.data_ptr(), B, L, C, stream)
    assert rc == 0, lib.fields_status_string(rc)
    return read, out


def test_noalloc_forward_matches_ordinary_forward_twice_in_a_row():
    from fields_lm_b200 import _lib
    lib = _lib.load()
    assert torch.cuda.is_available()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert lib.fields_read_static_scratch_bytes() == 16 << 20

    # two calls back to back on the shared buffer: different extents, different data
    for B, L, C, seed in ((2, 700, 512, 11), (3, 333, 132, 12)):
        args = _inputs(dev, B, L, C, seed)
        want_read, want_state = _ordinary(lib, *args, B, L, C, stream)
        got_read, got_state = _noalloc(lib, *args, B, L, C, stream)
        torch.cuda.synchronize()
        assert rel_err(got_read.cpu().numpy(), want_read.cpu().numpy()) < FP32_TOL
        assert rel_err(got_state.cpu().numpy(), want_state.cpu().numpy()) < FP32_TOL
        assert not bool(torch.isnan(got_read).any())


def test_noalloc_forward_allocates_nothing_and_covers_the_scalar_kernels():
    """The property the entry point exists for: after the first call on a device (which asks
    for the address of the built-in buffer), a call changes neither the driver's free memory
    nor the caching allocator's books. Also a channel count that is not a multiple of four
    (the three-phase scalar kernels on the shared buffer), and the per-device address on a
    second GPU where the box has one."""
    from fields_lm_b200 import _lib
    lib = _lib.load()
    devices = [0] + ([1] if torch.cuda.device_count() >= 2 else [])
    for index in devices:
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            B, L, C = 2, 257, 131
            args = _inputs(dev, B, L, C, 20 + index)
            want_read, want_state = _ordinary(lib, *args, B, L, C, stream)
            read = torch.empty(B, L, 4 * C, device=dev)
            out = torch.empty(B, 2 * C, device=dev)

            def call():
                rc = lib.fields_read_forward_noalloc(*[a.data_ptr() for a in args], read.data_ptr(),
                                                     out.data_ptr(), B, L, C, stream)
                assert rc == 0, lib.fields_status_string(rc)
                torch.cuda.synchronize(dev)
            call()                                        # first call on this device
            free_before, _ = torch.cuda.mem_get_info(dev)
            held_before = (torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev))
            call()
            free_after, _ = torch.cuda.mem_get_info(dev)
            assert free_after == free_before
            assert (torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)) == held_before
            assert rel_err(read.cpu().numpy(), want_read.cpu().numpy()) < FP32_TOL
            assert rel_err(out.cpu().numpy(), want_state.cpu().numpy()) < FP32_TOL


def test_noalloc_forward_refuses_extents_beyond_its_buffer():
    from fields_lm_b200 import _lib
    lib = _lib.load()
    B, L, C = 1, 65536, 512
    assert lib.fields_read_workspace_bytes(B, L, C, 0) > lib.fields_read_static_scratch_bytes()
    # refused before anything is dereferenced or launched, so placeholder pointers are safe
    rc = lib.fields_read_forward_noalloc(None, None, None, None, None, None, None, B, L, C, None)
    assert rc == 6
    assert b"static buffer" in lib.fields_status_string(rc)
