"""The tensor-core (tcgen05) restatement of the forward, an experiment on the bfloat16 boundary.

``fields_read_forward_bf16_tensor`` computes the intra-chunk sums as a product with a triangular
all-ones matrix on the tensor cores. It is held to the bfloat16 tolerance (2e-2 relative max-abs)
against the CPU oracle and against the production bfloat16 kernel.
"""
import numpy as np
import pytest
import torch

from conftest import BF16_TOL, rel_err
from oracle import field_oracle

pytestmark = pytest.mark.gpu


def _run(raw16, tr, ti, gm, state_in=None):
    from fields_lm_b200 import _lib
    lib = _lib.load()
    B, L, C3 = raw16.shape
    C = C3 // 3
    read = torch.empty(B, L, 4 * C, dtype=torch.bfloat16, device=raw16.device)
    state = torch.empty(B, 2 * C, device=raw16.device)
    err = torch.zeros(1, dtype=torch.int32, device=raw16.device)
    rc = lib.fields_read_forward_bf16_tensor(
        raw16.data_ptr(), tr.data_ptr(), ti.data_ptr(), gm.data_ptr(),
        None if state_in is None else state_in.data_ptr(), read.data_ptr(), state.data_ptr(),
        err.data_ptr(), B, L, C, torch.cuda.current_stream(raw16.device).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    return read, state


@pytest.mark.parametrize("B,L,C", [(2, 300, 64), (1, 128, 32), (3, 1000, 512), (2, 37, 20)])
def test_matches_the_oracle_within_the_bf16_tolerance(B, L, C):
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(B + L + C)
    radius = rng.uniform(0.5, 0.99995, C).astype(np.float32)
    theta = rng.uniform(-np.pi, np.pi, C).astype(np.float32)
    tr, ti = (radius * np.cos(theta)).astype(np.float32), (radius * np.sin(theta)).astype(np.float32)
    gm = np.sqrt(np.maximum(1 - radius ** 2, 1e-4)).astype(np.float32)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    raw[:, L // 3: L // 3 + 40, 2 * C:] = 30.0          # a stretch of saturated vacancy gates
    raw16 = torch.from_numpy(raw).bfloat16()
    s0 = rng.standard_normal((B, 2 * C)).astype(np.float32)
    t = [torch.from_numpy(a).to(dev) for a in (tr, ti, gm)]
    read, state = _run(raw16.to(dev), *t, state_in=torch.from_numpy(s0).to(dev))
    want, want_state = field_oracle.forward(raw16.float().numpy(), tr, ti, gm, state_in=s0)
    assert rel_err(read.float().cpu().numpy(), want) < BF16_TOL
    assert rel_err(state.cpu().numpy(), want_state) < BF16_TOL


def test_close_to_the_production_bf16_kernel_at_the_training_shape():
    from fields_lm_b200 import fused_field_read_bf16
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(1)
    B, L, C = 8, 2048, 512
    ring = torch.linspace(0.85, 0.999, C)
    theta = torch.linspace(0.03, torch.pi * 0.97, C)
    t = [(ring * torch.cos(theta)).to(dev), (ring * torch.sin(theta)).to(dev),
         torch.sqrt(1 - ring ** 2).to(dev)]
    raw16 = (torch.randn(B, L, 3 * C, generator=gen) * 0.577).bfloat16().to(dev)
    read, _ = _run(raw16, *t)
    with torch.no_grad():
        want = fused_field_read_bf16(raw16, *t)
    assert rel_err(read.float().cpu().numpy(), want.float().cpu().numpy()) < BF16_TOL
