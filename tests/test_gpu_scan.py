"""The real-valued scan on the GPU: the C ABI against the fixtures made by the reference's
``hierarchical_scan`` and against the oracle at the softpatch mixer's size, ``linear_scan``
(autograd) against the reference's function on the same GPU, and ``install_scan`` on the
reference's own softpatch mixer."""
import numpy as np
import pytest
import torch

import fields_lm_b200
from conftest import FP32_TOL, GOLDEN, rel_err
from fields_lm_b200 import _lib
from oracle import ref, scan_oracle

pytestmark = pytest.mark.gpu


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def _scan_c_abi(a, b, g, state_in=None, grad_state_out=None):
    """fields_scan_forward + fields_scan_backward on device buffers; ``a`` dense or per token."""
    lib = _lib.load()
    B, L, C = b.shape
    a_d, b_d, g_d = _dev(a), _dev(b), _dev(g)
    layout = (L, 1, 0) if a.ndim == 2 else (L * C, C, 1)
    sin = None if state_in is None else _dev(state_in)
    gso = None if grad_state_out is None else _dev(grad_state_out)
    states = torch.full((B, L, C), float("nan"), device="cuda")
    sout = torch.full((B, C), float("nan"), device="cuda")
    ga, gb = torch.full_like(states, float("nan")), torch.full_like(states, float("nan"))
    gsi = torch.full((B, C), float("nan"), device="cuda")
    n = lib.fields_scan_workspace_bytes(B, L, C)
    ws = torch.empty(max(n, 16), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    ptr = lambda t: None if t is None else t.data_ptr()
    rc = lib.fields_scan_forward(a_d.data_ptr(), *layout, b_d.data_ptr(), ptr(sin),
                                 states.data_ptr(), sout.data_ptr(), ws.data_ptr(), n, B, L, C, st)
    assert rc == 0, rc
    rc = lib.fields_scan_backward(a_d.data_ptr(), *layout, states.data_ptr(), ptr(sin),
                                  g_d.data_ptr(), ptr(gso), ga.data_ptr(), gb.data_ptr(),
                                  gsi.data_ptr(), ws.data_ptr(), n, B, L, C, st)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in (states, sout, ga, gb, gsi)]


@pytest.mark.parametrize("idx", range(6))
def test_c_abi_matches_the_reference_fixtures(idx):
    gold = np.load(GOLDEN / "scan_small.npz")
    name = str(gold["cases"][idx])
    c = {k: gold[f"{name}/{k}"] for k in ("a", "b", "grad_states", "states", "grad_a", "grad_b")}
    states, sout, ga, gb, _ = _scan_c_abi(c["a"], c["b"], c["grad_states"])
    assert rel_err(states, c["states"]) < FP32_TOL
    np.testing.assert_array_equal(sout, states[:, -1])
    if c["a"].ndim == 2:
        ga = ga.astype(np.float64).sum(axis=2)
    assert rel_err(gb, c["grad_b"]) < FP32_TOL
    assert rel_err(ga, c["grad_a"]) < FP32_TOL


@pytest.mark.parametrize("B,L,C,per_token", [(8, 2048, 64, True), (2, 4097, 33, False),
                                              (1, 65536, 64, True)])
def test_c_abi_matches_the_oracle_at_size(B, L, C, per_token):
    """The softpatch mixer's size (8 x 2,048 tokens, rank 64, one decay per token), a ragged
    dense case, and a 65,536-token sequence; with states in and out."""
    rng = np.random.default_rng(L + C)
    a = rng.uniform(0.01, 0.99, (B, L) if per_token else (B, L, C)).astype(np.float32)
    b = rng.standard_normal((B, L, C)).astype(np.float32)
    g = rng.standard_normal((B, L, C)).astype(np.float32)
    sin = rng.standard_normal((B, C)).astype(np.float32)
    gso = rng.standard_normal((B, C)).astype(np.float32)
    wide = a[..., None] if per_token else a
    want, want_last = scan_oracle.forward(wide, b, sin)
    wa, wb, wsi = scan_oracle.backward(wide, b, g, sin, gso)
    states, sout, ga, gb, gsi = _scan_c_abi(a, b, g, sin, gso)
    assert rel_err(states, want) < FP32_TOL and rel_err(sout, want_last) < FP32_TOL
    assert rel_err(gb, wb) < FP32_TOL and rel_err(ga, wa) < FP32_TOL
    assert rel_err(gsi, wsi) < FP32_TOL


def test_results_are_bitwise_reproducible():
    rng = np.random.default_rng(3)
    a = rng.uniform(0.01, 0.99, (4, 700)).astype(np.float32)
    b = rng.standard_normal((4, 700, 64)).astype(np.float32)
    g = rng.standard_normal((4, 700, 64)).astype(np.float32)
    first = _scan_c_abi(a, b, g)
    again = _scan_c_abi(a, b, g)
    for x, y in zip(first[:4], again[:4]):
        np.testing.assert_array_equal(x, y)


@pytest.mark.skipif(not ref.available(), reason="staged reference absent")
def test_linear_scan_equals_the_reference_function_on_the_same_gpu():
    """``hierarchical_scan`` of the staged reference (PyTorch ops, CUDA) and ``linear_scan`` on
    the same tensors, built the way the softpatch mixer builds them (expanded decay)."""
    canon = ref.load_canon()
    gen = torch.Generator().manual_seed(7)
    B, L, R = 4, 1500, 64
    boundary0 = torch.rand(B, L, generator=gen).clamp(0.01, 0.99).cuda()
    z0 = torch.randn(B, L, R, generator=gen).cuda()
    g = torch.randn(B, L, R, generator=gen).cuda()
    results = []
    for fn in (canon.hierarchical_scan, fields_lm_b200.linear_scan):
        boundary = boundary0.clone().requires_grad_(True)
        z = z0.clone().requires_grad_(True)
        a = (1.0 - boundary)[..., None].expand_as(z)
        state = fn(a, boundary[..., None] * z, block=32)
        state.backward(g)
        results.append([t.detach().cpu().numpy() for t in (state, boundary.grad, z.grad)])
    for got, want, name in zip(results[1], results[0], ("state", "grad_boundary", "grad_z")):
        assert rel_err(got, want) < FP32_TOL, name


def test_linear_scan_argument_errors():
    a = torch.rand(1, 8, 4, device="cuda")
    with pytest.raises(ValueError, match="field_chunk"):
        fields_lm_b200.linear_scan(a, a, block=65)
    with pytest.raises(RuntimeError, match="CUDA"):
        fields_lm_b200.linear_scan(a.cpu(), a.cpu())
    with pytest.raises(TypeError):
        fields_lm_b200.linear_scan(a.double(), a.double())
    with pytest.raises(ValueError):
        fields_lm_b200.linear_scan(a, a[:, :4])


@pytest.mark.skipif(not ref.available(), reason="staged reference absent")
def test_scan_entry_hands_other_calls_to_the_original():
    """The replacement global keeps the complex CPU call of ``reference_field_read`` on the
    reference's own function."""
    from fields_lm_b200.scan import scan_entry
    canon = ref.load_canon()
    calls = []

    def original(a, b, block=32):
        calls.append(a.dtype)
        return canon.hierarchical_scan(a, b, block)

    entry = scan_entry(original)
    a = torch.rand(1, 40, 3, dtype=torch.complex64)
    out = entry(a, a, 32)
    assert calls == [torch.complex64] and out.dtype == torch.complex64
    real = torch.rand(1, 40, 3, device="cuda")
    entry(real, real, block=32)
    assert calls == [torch.complex64]          # the CUDA fp32 call did not reach the original
