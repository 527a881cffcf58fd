"""The reference's full 24-layer model with the CUDA library swapped in (GPU).

``build_official_fields`` of the staged reference builds the promoted 18 Field / 2 Mamba-2 /
4 refresh model; one training step under bf16 autocast runs first with the reference's Triton
Field kernels, then with ``fields_lm_b200.install(model)`` on the same object. The Mamba-2
editors are the labelled stand-in of ``oracle/mamba_standin.py`` on both sides where
``mamba-ssm`` is not installed. Smaller batch than the benchmark's [8, 2048] to keep the test
short; the benchmark's ``full_model`` leg runs the full shape.
"""
import pytest
import torch

import fields_lm_b200
from conftest import BF16_TOL, FP32_TOL
from oracle import full_model, ref

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref.available(), reason="staged reference absent")]


def test_training_step_matches_the_reference_triton_path():
    device = torch.device("cuda", 0)
    model, _ = full_model.build(device, model_seed=0)
    model.train()
    audit = model.topology_audit
    assert (audit["native_field_count"], audit["mamba_count"], audit["refresh_count"]) == (18, 2, 4)
    ids, labels = full_model.token_batch(2, 1024, 11, device)

    loss_ref = float(full_model.training_step(model, ids, labels))
    grads_ref = full_model.gradients(model)
    reads_ref = full_model.reads_by_block(model, ids)
    # the floor: the reference against itself with another chunk length (32 instead of 64)
    full_model.set_triton_geometry(model, 32, 32)
    full_model.training_step(model, ids, labels)
    floor, _ = full_model.compare_gradients(full_model.gradients(model), grads_ref)
    floor_norm, _ = full_model.norm_relative(full_model.gradients(model), grads_ref)
    full_model.set_triton_geometry(model, 32, 64)

    # one module namespace for all 18 blocks; the softpatch mixer's scan goes along
    assert fields_lm_b200.install(model, scan=True) == 1
    try:
        loss_new = float(full_model.training_step(model, ids, labels))
        grads_new = full_model.gradients(model)
        reads_new = full_model.reads_by_block(model, ids)
    finally:
        fields_lm_b200.uninstall(model)
    assert set(grads_new) == set(grads_ref) and len(reads_new) == len(reads_ref) == 18
    assert all(torch.isfinite(g).all() for g in grads_new.values())
    # the first Field block sees identical inputs on both sides: operator-level parity in situ
    first = float((reads_new[0] - reads_ref[0]).abs().max() / reads_ref[0].abs().max())
    assert first < FP32_TOL, first
    assert abs(loss_new - loss_ref) <= BF16_TOL * abs(loss_ref)
    worst_norm, where_norm = full_model.norm_relative(grads_new, grads_ref)
    assert worst_norm <= max(BF16_TOL, 3 * floor_norm), (worst_norm, where_norm, floor_norm)
    # element-wise max error: single bfloat16 flips in 24 stacked layers move individual
    # gradient entries; held to what the reference's own second geometry does to them
    worst, where = full_model.compare_gradients(grads_new, grads_ref)
    assert worst <= max(BF16_TOL, 3 * floor), (worst, where, floor)


def test_softpatch_mixer_with_the_scan_installed():
    """The reference's ``FastBoundaryStateMixer`` of the built model (block 11's softpatch: a
    learned boundary score, a rank-64 real scan, an up projection), fp32, first on the
    reference's ``hierarchical_scan`` then with ``install_scan``: output and all gradients."""
    device = torch.device("cuda", 0)
    model, _ = full_model.build(device, model_seed=0)
    mixer = model.core_model.softpatch
    assert type(mixer).__name__ == "FastBoundaryStateMixer"
    gen = torch.Generator().manual_seed(21)
    dim = mixer.down.in_features
    x0 = torch.randn(2, 700, dim, generator=gen).to(device)
    gy = torch.randn(2, 700, dim, generator=gen).to(device)
    tokens = torch.randint(0, 16384, (2, 700), generator=gen).to(device)

    def run():
        mixer.zero_grad(set_to_none=True)
        x = x0.clone().requires_grad_(True)
        y = mixer(x, tokens)
        y.backward(gy)
        return [y.detach(), x.grad] + [p.grad for p in mixer.parameters() if p.grad is not None]

    want = run()
    assert fields_lm_b200.install_scan(model) == 1
    try:
        got = run()
    finally:
        fields_lm_b200.uninstall(model)
    again = run()                                  # the original is back
    assert len(got) == len(want) >= 5
    for a, b in zip(got, want):
        assert float((a - b).abs().max()) <= 2e-5 * float(b.abs().max())
    for a, b in zip(again, want):
        assert float((a - b).abs().max()) <= 1e-6 * float(b.abs().max())
