"""The pinned-host pipeline gives the same results as one device-resident call."""
import numpy as np
import pytest
import torch

from conftest import FP32_TOL, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows", [1, 3])
def test_host_pipeline_matches_device_call(rows):
    from fields_lm_b200 import fused_field_read
    from fields_lm_b200.host import HostFieldRead
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(21)
    B, L, C = 5, 300, 128
    radius = torch.rand(C, generator=gen) * 0.49 + 0.5
    theta = (torch.rand(C, generator=gen) * 2 - 1) * torch.pi
    tr, ti = (radius * torch.cos(theta)).to(dev), (radius * torch.sin(theta)).to(dev)
    gm = torch.sqrt(1 - radius ** 2).to(dev)
    raw = torch.randn(B, L, 3 * C, generator=gen).pin_memory()
    grad = torch.randn(B, L, 4 * C, generator=gen).pin_memory()
    read = torch.empty(B, L, 4 * C).pin_memory()
    graw = torch.empty(B, L, 3 * C).pin_memory()

    pipe = HostFieldRead(dev, B, L, C, rows_per_chunk=rows)
    for _ in range(2):  # second call reuses slots and events
        gpar = pipe.fwd_bwd(raw, grad, tr, ti, gm, read, graw).clone()
        torch.cuda.synchronize()

    p = [t.clone().requires_grad_(True) for t in (tr, ti, gm)]
    r = raw.to(dev).requires_grad_(True)
    want = fused_field_read(r, *p, 32, 64)
    want.backward(grad.to(dev))
    assert rel_err(read.numpy(), want.detach().cpu().numpy()) < FP32_TOL
    assert rel_err(graw.numpy(), r.grad.cpu().numpy()) < FP32_TOL
    for k in range(3):
        assert rel_err(gpar[k].cpu().numpy(), p[k].grad.cpu().numpy()) < FP32_TOL


def test_host_pipeline_calls_may_overlap():
    """wait=False: three calls on different inputs issued back to back, one join; every call's
    outputs (host tensors of its own) equal the device-resident result."""
    from fields_lm_b200 import fused_field_read
    from fields_lm_b200.host import HostFieldRead
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(23)
    B, L, C = 4, 200, 128
    radius = torch.rand(C, generator=gen) * 0.49 + 0.5
    theta = (torch.rand(C, generator=gen) * 2 - 1) * torch.pi
    tr, ti = (radius * torch.cos(theta)).to(dev), (radius * torch.sin(theta)).to(dev)
    gm = torch.sqrt(1 - radius ** 2).to(dev)
    pipe = HostFieldRead(dev, B, L, C, rows_per_chunk=1)
    calls = []
    for _ in range(3):
        raw = torch.randn(B, L, 3 * C, generator=gen).pin_memory()
        grad = torch.randn(B, L, 4 * C, generator=gen).pin_memory()
        read = torch.empty(B, L, 4 * C).pin_memory()
        graw = torch.empty(B, L, 3 * C).pin_memory()
        gpar = torch.empty(3, C).pin_memory()
        pipe.fwd_bwd(raw, grad, tr, ti, gm, read, graw, gpar_host=gpar, wait=False)
        calls.append((raw, grad, read, graw, gpar))
    pipe.join()
    torch.cuda.synchronize()
    for raw, grad, read, graw, gpar in calls:
        p = [t.clone().requires_grad_(True) for t in (tr, ti, gm)]
        r = raw.to(dev).requires_grad_(True)
        want = fused_field_read(r, *p, 32, 64)
        want.backward(grad.to(dev))
        assert rel_err(read.numpy(), want.detach().cpu().numpy()) < FP32_TOL
        assert rel_err(graw.numpy(), r.grad.cpu().numpy()) < FP32_TOL
        for k in range(3):
            assert rel_err(gpar[k].numpy(), p[k].grad.cpu().numpy()) < FP32_TOL
