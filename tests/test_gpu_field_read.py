"""GPU parity tests of the CUDA operator against the CPU oracle and the reference fixtures.

Every call goes through the C ABI (ctypes) of libfields_read.so, either directly
or through the autograd function. Tolerances: 1e-5 relative for fp32 (FP32_TOL),
2e-2 relative max-abs for bf16 activations with an fp32 state (BF16_TOL), with
relative error = max|x - ref| / max(max|ref|, 1e-6).
"""
import numpy as np
import pytest
import torch

from conftest import BF16_TOL, FP32_TOL, rel_err
from oracle import field_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["product", "walk", "single_pass", "three_phase"])
def algo(request, monkeypatch):
    """Every test runs on the product library and, through the test build of the same source
    (which reads the variable at each call), on every kernel family."""
    if request.param == "product":
        return "single_pass"
    request.getfixturevalue("variants_library")
    monkeypatch.setenv("FIELDS_READ_ALGO", request.param)
    return request.param


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda", 0)


def _params(C, rng):
    radius = rng.uniform(0.5, 0.99995, C).astype(np.float32)
    theta = rng.uniform(-np.pi, np.pi, C).astype(np.float32)
    return ((radius * np.cos(theta)).astype(np.float32),
            (radius * np.sin(theta)).astype(np.float32),
            np.sqrt(np.maximum(1 - radius ** 2, 1e-4)).astype(np.float32))


def _init_params(C):
    ring = np.linspace(0.85, 0.999, C, dtype=np.float32)
    theta = np.linspace(0.03, np.pi * 0.97, C, dtype=np.float32)
    return ((ring * np.cos(theta)).astype(np.float32), (ring * np.sin(theta)).astype(np.float32),
            np.sqrt(np.maximum(1 - ring ** 2, 1e-4)).astype(np.float32))


def _t(x, dev, grad=False):
    return None if x is None else torch.from_numpy(np.ascontiguousarray(x)).to(dev).requires_grad_(grad)


def run_op(dev, raw, tr, ti, gm, grad_read=None, state_in=None, grad_state_out=None):
    """Forward (+ backward when grad_read is given) on the GPU through autograd."""
    from fields_lm_b200 import field_read_with_state
    need = grad_read is not None
    raw_t, tr_t, ti_t, gm_t = (_t(a, dev, need) for a in (raw, tr, ti, gm))
    sin_t = _t(state_in, dev, need)
    read, state = field_read_with_state(raw_t, tr_t, ti_t, gm_t, sin_t)
    out = {"read": read.detach().cpu().numpy(), "state": state.detach().cpu().numpy()}
    if need:
        outs, grads = [read], [_t(grad_read, dev)]
        if grad_state_out is not None:
            outs.append(state)
            grads.append(_t(grad_state_out, dev))
        torch.autograd.backward(outs, grads)
        out.update(grad_raw=raw_t.grad.cpu().numpy(), grad_tr=tr_t.grad.cpu().numpy(),
                   grad_ti=ti_t.grad.cpu().numpy(), grad_gamma=gm_t.grad.cpu().numpy())
        if sin_t is not None:
            out["grad_state_in"] = sin_t.grad.cpu().numpy()
    return out


def check_against_oracle(dev, raw, tr, ti, gm, grad_read, state_in=None, grad_state_out=None,
                         tol=FP32_TOL):
    got = run_op(dev, raw, tr, ti, gm, grad_read, state_in, grad_state_out)
    ref_read, ref_state = field_oracle.forward(raw, tr, ti, gm, state_in=state_in)
    assert rel_err(got["read"], ref_read) < tol
    assert rel_err(got["state"], ref_state) < tol
    ref = field_oracle.backward(raw, tr, ti, gm, grad_read, state_in=state_in,
                                grad_state_out=grad_state_out)
    for name, r in zip(("grad_raw", "grad_tr", "grad_ti", "grad_gamma"), ref):
        assert rel_err(got[name], r) < tol, name
    if state_in is not None:
        assert rel_err(got["grad_state_in"], ref[4]) < tol


def test_library_is_loaded_from_the_tree():
    from fields_lm_b200 import _lib
    _lib.load()
    with open("/proc/self/maps") as f:
        assert "libfields_read" in f.read()


def test_golden_small_cases(dev, golden_small):
    for name in golden_small["cases"]:
        c = {k: golden_small[f"{name}/{k}"] for k in
             ("raw", "tr", "ti", "gamma", "grad_read", "read", "grad_raw", "grad_tr", "grad_ti",
              "grad_gamma")}
        got = run_op(dev, c["raw"], c["tr"], c["ti"], c["gamma"], c["grad_read"])
        for key in ("read", "grad_raw", "grad_tr", "grad_ti", "grad_gamma"):
            assert rel_err(got[key], c[key]) < FP32_TOL, (name, key)


def test_golden_config1_operator(dev, golden_config1):
    g = golden_config1
    steps = g["steps"]
    got = run_op(dev, g["raw"], g["tr"], g["ti"], g["gamma"], g["grad_read"].astype(np.float32))
    assert rel_err(got["read"][:, steps], g["read_steps"]) < FP32_TOL
    assert rel_err(got["grad_raw"][:, steps], g["grad_raw_steps"]) < FP32_TOL
    for key in ("grad_tr", "grad_ti", "grad_gamma"):
        assert rel_err(got[key], g[key]) < FP32_TOL, key


@pytest.mark.parametrize("L", [1, 37, 63, 64, 65, 2048])
@pytest.mark.parametrize("C", [512, 20, 7])
def test_shape_sweep(dev, L, C):
    rng = np.random.default_rng(L * 31 + C)
    B = 2 if L < 2048 else 1
    tr, ti, gm = _params(C, rng)
    raw = (rng.standard_normal((B, L, 3 * C)) * 1.5).astype(np.float32)
    grad_read = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    check_against_oracle(dev, raw, tr, ti, gm, grad_read)


@pytest.mark.parametrize("variant", ["1", "2", "3"])
def test_single_pass_alternatives(dev, algo, monkeypatch, variant, request):
    """The selectable alternatives of the single-pass kernels (tile shapes, two-sweep forward,
    backward with recomputed states, tile-resident backward) against the oracle."""
    if algo != "single_pass":
        pytest.skip("variants exist for the single-pass kernels only")
    request.getfixturevalue("variants_library")
    monkeypatch.setenv("FIELDS_FWD_VARIANT", variant)
    monkeypatch.setenv("FIELDS_BWD_VARIANT", variant)
    rng = np.random.default_rng(int(variant))
    for B, L, C, with_state in ((2, 300, 512, False), (1, 2053, 132, True), (3, 17, 20, True)):
        tr, ti, gm = _params(C, rng)
        raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
        grad_read = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
        s_in = rng.standard_normal((B, 2 * C)).astype(np.float32) if with_state else None
        g_out = rng.standard_normal((B, 2 * C)).astype(np.float32) if with_state else None
        check_against_oracle(dev, raw, tr, ti, gm, grad_read, s_in, g_out)


@pytest.mark.parametrize("B,L,C", [(2, 300, 512), (1, 2053, 132), (2, 8, 20), (3, 9, 4)])
def test_lean_backward_keeps_state_rows_only(dev, B, L, C):
    """lean=True: the autograd function keeps every eighth state row instead of `read`; gradients
    equal the oracle's and the ordinary backward's."""
    from fields_lm_b200 import field_read_with_state
    rng = np.random.default_rng(L + C)
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    grad = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    s_in = rng.standard_normal((B, 2 * C)).astype(np.float32)
    g_out = rng.standard_normal((B, 2 * C)).astype(np.float32)
    raw_t, tr_t, ti_t, gm_t, sin_t = (_t(a, dev, True) for a in (raw, tr, ti, gm, s_in))
    read, state = field_read_with_state(raw_t, tr_t, ti_t, gm_t, sin_t, lean=True)
    saved = read.grad_fn.saved_tensors if hasattr(read.grad_fn, "saved_tensors") else ()
    assert all(t.numel() < read.numel() or t.shape[-1] == 3 * C for t in saved)
    torch.autograd.backward([read, state], [_t(grad, dev), _t(g_out, dev)])
    want = field_oracle.backward(raw, tr, ti, gm, grad, state_in=s_in, grad_state_out=g_out)
    got = (raw_t.grad, tr_t.grad, ti_t.grad, gm_t.grad, sin_t.grad)
    for g, w in zip(got, want):
        assert rel_err(g.cpu().numpy(), w) < FP32_TOL


def test_saturated_gates_and_slowest_decay(dev):
    """Inputs that drive tanh and sigmoid into saturation, zero inputs, and every channel at the
    largest radius the mixer allows (0.99995, 4,096 steps of accumulation), against the oracle."""
    rng = np.random.default_rng(99)
    B, L, C = 2, 4096, 128
    radius = np.full(C, 0.99995, np.float32)
    theta = np.linspace(0.03, np.pi * 0.97, C).astype(np.float32)
    tr, ti = radius * np.cos(theta), radius * np.sin(theta)
    gm = np.sqrt(np.maximum(1 - radius ** 2, 1e-4)).astype(np.float32)
    raw = (rng.standard_normal((B, L, 3 * C)) * 8.0).astype(np.float32)
    raw[:, 100:200] = 0.0          # a stretch of exact zeros
    raw[:, 300:400, 2 * C:] = -60  # vacancy 0: pure decay; then +60: vacancy at its maximum
    raw[:, 400:500, 2 * C:] = 60
    grad_read = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    check_against_oracle(dev, raw, tr, ti, gm, grad_read)


def test_state_in_and_out(dev):
    rng = np.random.default_rng(77)
    B, L, C = 3, 200, 132
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    grad_read = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    s_in = rng.standard_normal((B, 2 * C)).astype(np.float32)
    g_out = rng.standard_normal((B, 2 * C)).astype(np.float32)
    check_against_oracle(dev, raw, tr, ti, gm, grad_read, s_in, g_out)


def test_spans_chain_exactly_like_one_pass(dev):
    """Causality: a sequence cut into spans that hand over the state equals one pass."""
    rng = np.random.default_rng(5)
    B, L, C = 2, 1000, 512
    tr, ti, gm = _init_params(C)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    full = run_op(dev, raw, tr, ti, gm)
    state, parts = None, []
    for lo, hi in ((0, 333), (333, 334), (334, 1000)):
        out = run_op(dev, raw[:, lo:hi], tr, ti, gm, state_in=state)
        parts.append(out["read"])
        state = out["state"]
    assert rel_err(np.concatenate(parts, 1), full["read"]) < 2e-6
    assert rel_err(state, full["state"]) < 2e-6
    # a prefix does not depend on what follows it
    prefix = run_op(dev, raw[:, :517], tr, ti, gm)
    assert rel_err(prefix["read"], full["read"][:, :517]) < 2e-6


@pytest.mark.parametrize("C", [512, 20, 7])
def test_backward_over_spans_equals_one_backward_pass(dev, C):
    """The device operations of the sequence-sharded backward, spans taken one after another on
    one GPU: dual summaries folded in reverse order hand every span the carry of a single pass."""
    from fields_lm_b200.seqpar import CudaOps
    ops = CudaOps()
    rng = np.random.default_rng(17 + C)
    B, L = 2, 700
    tr, ti, gm = _init_params(C)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    grad = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    want = field_oracle.backward(raw, tr, ti, gm, grad)
    t = lambda a: _t(np.ascontiguousarray(a), dev)
    tr_t, ti_t, gm_t = t(tr), t(ti), t(gm)
    spans = [(0, 233), (233, 234), (234, 700)]
    fwd = torch.stack([ops.span_summary(t(raw[:, a:b]), tr_t, ti_t, gm_t) for a, b in spans])
    dual = torch.stack([ops.span_summary_backward(t(raw[:, a:b]), tr_t, ti_t, t(grad[:, a:b]))
                        for a, b in spans])
    g_raw = np.zeros_like(raw)
    g_par = np.zeros((3, C))
    for r, (a, b) in enumerate(spans):
        state_in = ops.fold(fwd, r, None)
        carry = ops.fold_backward(dual, r, None)
        read, _ = ops.forward(t(raw[:, a:b]), tr_t, ti_t, gm_t, state_in)
        gr, gp, _ = ops.backward(t(raw[:, a:b]), tr_t, ti_t, gm_t, read, t(grad[:, a:b]), state_in,
                                 carry)
        g_raw[:, a:b] = gr.cpu().numpy()
        g_par += gp.double().cpu().numpy()
    assert rel_err(g_raw, want[0]) < FP32_TOL
    for k in range(3):
        assert rel_err(g_par[k], want[1 + k]) < FP32_TOL


def test_ordinary_launches_give_the_same_results(dev, monkeypatch, variants_library):
    """FIELDS_READ_PDL=0: plain launches and a memset instead of dependent launches and the fill
    kernel (the test build reads the variable per call; the product library once)."""
    monkeypatch.setenv("FIELDS_READ_PDL", "0")
    rng = np.random.default_rng(77)
    B, L, C = 2, 300, 512
    tr, ti, gm = _init_params(C)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    grad = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    check_against_oracle(dev, raw, tr, ti, gm, grad)


def test_tiles_handed_out_by_ticket_give_the_same_results(dev, monkeypatch, variants_library):
    """FIELDS_TILE_TICKET=1 (test build): blocks take their tile from a counter in the workspace
    header instead of their block index, so no tile waits for a block that has not started,
    whatever order the hardware dispatches blocks in. Several waves of tiles per chain."""
    monkeypatch.setenv("FIELDS_TILE_TICKET", "1")
    rng = np.random.default_rng(78)
    for B, L, C in ((2, 4500, 512), (3, 70, 132)):
        tr, ti, gm = _init_params(C)
        raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
        grad = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
        check_against_oracle(dev, raw, tr, ti, gm, grad)


def _config2_inputs(B=8, L=2048, C=512):
    """bf16-rounded activations held in fp32, as autocast hands them to the operator."""
    gen = torch.Generator().manual_seed(1)
    raw = (torch.randn(B, L, 3 * C, generator=gen) * 0.577).bfloat16().float().numpy()
    grad_read = torch.randn(B, L, 4 * C, generator=gen).bfloat16().float().numpy()
    return raw, grad_read


def test_config2_full_size_forward_backward(dev):
    """Batch 8 x 2,048 tokens, C = 512: the training configuration, against the oracle."""
    raw, grad_read = _config2_inputs()
    tr, ti, gm = _init_params(512)
    check_against_oracle(dev, raw, tr, ti, gm, grad_read)


def test_config4_full_size_forward(dev):
    """Batch 1 x 65,536 tokens forward, against the oracle."""
    gen = torch.Generator().manual_seed(2)
    raw = (torch.randn(1, 65536, 1536, generator=gen) * 0.577).bfloat16().float().numpy()
    tr, ti, gm = _init_params(512)
    got = run_op(dev, raw, tr, ti, gm)
    ref, ref_state = field_oracle.forward(raw, tr, ti, gm)
    assert rel_err(got["read"], ref) < FP32_TOL
    assert rel_err(got["state"], ref_state) < FP32_TOL


def test_run_to_run_reproducibility(dev, algo):
    """The chain-walking and three-phase kernels are bitwise reproducible. The single-pass
    kernels compose whatever aggregates have been published when a block looks back, so the
    association of the floating-point products depends on timing: equal to rounding only."""
    raw, grad_read = _config2_inputs(B=2, L=777)
    tr, ti, gm = _init_params(512)
    a = run_op(dev, raw, tr, ti, gm, grad_read)
    b = run_op(dev, raw, tr, ti, gm, grad_read)
    for key in a:
        if algo == "single_pass":
            assert rel_err(a[key], b[key]) < 2e-6, key
        else:
            np.testing.assert_array_equal(a[key], b[key])


def test_outputs_stay_inside_their_buffers(dev, algo):
    """Direct C-ABI call with sentinel guard bands around every output and the workspace."""
    from fields_lm_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(1)
    B, L, C = 2, 150, 36
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    grad_read = rng.standard_normal((B, L, 4 * C)).astype(np.float32)
    PAD, SENT = 256, 1234.5

    def guarded(n):
        buf = torch.full((n + 2 * PAD,), SENT, device=dev, dtype=torch.float32)
        return buf, buf[PAD:PAD + n]

    def intact(buf, n):
        return bool((buf[:PAD] == SENT).all() and (buf[PAD + n:] == SENT).all())

    t = {k: _t(v, dev) for k, v in dict(raw=raw, tr=tr, ti=ti, gm=gm, grad_read=grad_read).items()}
    n_read, n_raw = B * L * 4 * C, B * L * 3 * C
    read_buf, read = guarded(n_read)
    state_buf, state = guarded(B * 2 * C)
    wsf = lib.fields_read_workspace_bytes(B, L, C, 0)
    ws_buf, ws = guarded(wsf // 4)
    s = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.fields_read_forward(t["raw"].data_ptr(), t["tr"].data_ptr(), t["ti"].data_ptr(),
                                 t["gm"].data_ptr(), None, read.data_ptr(), state.data_ptr(),
                                 ws.data_ptr(), wsf, B, L, C, s)
    assert rc == 0
    if algo == "single_pass":  # the error word exists only in the single-pass workspace layout
        assert lib.fields_read_device_status(ws.data_ptr(), s) == 0
    torch.cuda.synchronize()
    assert intact(read_buf, n_read) and intact(state_buf, B * 2 * C) and intact(ws_buf, wsf // 4)
    ref, _ = field_oracle.forward(raw, tr, ti, gm)
    assert rel_err(read.cpu().numpy().reshape(B, L, 4 * C), ref) < FP32_TOL

    graw_buf, graw = guarded(n_raw)
    gp_buf, gp = guarded(3 * C)
    wsb = lib.fields_read_workspace_bytes(B, L, C, 1)
    wsb_buf, wsb_t = guarded(wsb // 4)
    rc = lib.fields_read_backward(t["raw"].data_ptr(), t["tr"].data_ptr(), t["ti"].data_ptr(),
                                  t["gm"].data_ptr(), None, read.data_ptr(),
                                  t["grad_read"].data_ptr(), None, graw.data_ptr(),
                                  gp[:C].data_ptr(), gp[C:2 * C].data_ptr(), gp[2 * C:].data_ptr(),
                                  None, wsb_t.data_ptr(), wsb, B, L, C, s)
    assert rc == 0
    if algo == "single_pass":
        assert lib.fields_read_device_status(wsb_t.data_ptr(), s) == 0
    torch.cuda.synchronize()
    assert intact(graw_buf, n_raw) and intact(gp_buf, 3 * C) and intact(wsb_buf, wsb // 4)
    # too-small workspace and null pointers are refused with a status, nothing is launched
    assert lib.fields_read_forward(t["raw"].data_ptr(), t["tr"].data_ptr(), t["ti"].data_ptr(),
                                   t["gm"].data_ptr(), None, read.data_ptr(), None,
                                   ws.data_ptr(), wsf - 4, B, L, C, s) == 2
    assert lib.fields_read_forward(None, t["tr"].data_ptr(), t["ti"].data_ptr(),
                                   t["gm"].data_ptr(), None, read.data_ptr(), None,
                                   ws.data_ptr(), wsf, B, L, C, s) == 1


def test_unaligned_views_take_the_scalar_path(dev):
    """A raw tensor that starts 4 bytes off a 16-byte boundary still gives the same answer."""
    from fields_lm_b200 import fused_field_read
    rng = np.random.default_rng(2)
    B, L, C = 1, 90, 64
    tr, ti, gm = _params(C, rng)
    raw = rng.standard_normal((B, L, 3 * C)).astype(np.float32)
    store = torch.zeros(raw.size + 1, device=dev)
    store[1:] = _t(raw.ravel(), dev)
    shifted = store[1:].view(B, L, 3 * C)
    assert shifted.data_ptr() % 16 == 4
    a = fused_field_read(shifted, _t(tr, dev), _t(ti, dev), _t(gm, dev), 32, 64)
    b = fused_field_read(_t(raw, dev), _t(tr, dev), _t(ti, dev), _t(gm, dev), 32, 64)
    # same arithmetic, but the two instantiations may contract multiply-adds differently
    assert rel_err(a.cpu().numpy(), b.cpu().numpy()) < 1e-6


def test_wrong_dtype_and_shape_raise_like_the_reference(dev):
    from fields_lm_b200 import fused_field_read
    p = torch.zeros(4, device=dev)
    with pytest.raises(TypeError, match="raw must be float32"):
        fused_field_read(torch.zeros(1, 2, 12, device=dev, dtype=torch.bfloat16), p, p, p, 32, 64)
    with pytest.raises(ValueError):
        fused_field_read(torch.zeros(1, 2, 13, device=dev), p, p, p, 32, 64)
    with pytest.raises(ValueError):
        fused_field_read(torch.zeros(1, 2, 15, device=dev), p, p, p, 32, 64)


def test_empty_sequence(dev):
    from fields_lm_b200 import field_read_with_state
    p = torch.ones(4, device=dev)
    s = torch.full((2, 8), 3.0, device=dev)
    read, state = field_read_with_state(torch.zeros(2, 0, 12, device=dev), p, p, p, s)
    assert read.shape == (2, 0, 16)
    assert bool((state == 3.0).all())


def test_a_wait_that_nothing_satisfies_ends_with_a_timeout_status(dev):
    """Bounded wait: a block waiting for a publication that never comes gives up after its poll
    limit, reports FIELDS_ERR_TIMEOUT through the error word, and the GPU stays usable."""
    from fields_lm_b200 import _lib
    lib = _lib.load()
    ws = torch.empty(16384, dtype=torch.uint8, device=dev)
    s = torch.cuda.current_stream(dev).cuda_stream
    assert lib.fields_read_selftest_wait(ws.data_ptr(), ws.numel(), 2000, s) == 4
    out = ws[256 + 4 * 128 * 16 + 4 * 128 * 8:][:128 * 2 * 4].view(torch.float32)
    assert bool(torch.isnan(out).all())
    # the context is intact: an ordinary call still works afterwards
    p = torch.ones(4, device=dev) * 0.5
    from fields_lm_b200 import fused_field_read
    y = fused_field_read(torch.zeros(1, 3, 12, device=dev), p, p, p, 32, 64)
    assert bool(torch.isfinite(y).all())


def test_bf16_boundary_against_oracle(dev):
    """bfloat16 raw / read / gradients with an fp32 state: 2e-2 relative max-abs (BF16_TOL)."""
    from fields_lm_b200 import fused_field_read_bf16
    gen = torch.Generator().manual_seed(31)
    B, L, C = 4, 1024, 512
    tr, ti, gm = _init_params(C)
    raw = (torch.randn(B, L, 3 * C, generator=gen) * 0.577).bfloat16()
    grad = torch.randn(B, L, 4 * C, generator=gen).bfloat16()
    t = [_t(a, dev, True) for a in (tr, ti, gm)]
    r = raw.to(dev).requires_grad_(True)
    read = fused_field_read_bf16(r, *t)
    assert read.dtype == torch.bfloat16
    read.backward(grad.to(dev))
    rawf, gradf = raw.float().numpy(), grad.float().numpy()
    ref_read, _ = field_oracle.forward(rawf, tr, ti, gm)
    ref = field_oracle.backward(rawf, tr, ti, gm, gradf)
    assert rel_err(read.detach().float().cpu().numpy(), ref_read) < 2 ** -7
    assert rel_err(r.grad.float().cpu().numpy(), ref[0]) < BF16_TOL
    for k in range(3):
        assert rel_err(t[k].grad.cpu().numpy(), ref[k + 1]) < BF16_TOL
