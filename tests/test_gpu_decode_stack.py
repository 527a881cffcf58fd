"""Recurrent decode at the stated size: 18 Field blocks, d_model 1,024, batch 256, a 2,048-token
prefix of seeded ids, then single-token steps (GPU).

The oracle is the staged reference itself: its ``FieldBlock`` stack with ``backend="reference"``
run on the CPU over prefix + steps tokens in one full-sequence pass (the reference has no
incremental path; the stack is causal). The CPU side runs a few of the 256 sequences - the
same ids and the same seeded weights - which is all the comparison needs, since sequences never
mix. Step outputs must equal the full pass at the new positions, and the carried state of every
block must equal the state planes of that block's ``read`` there.
"""
import pytest
import torch

from conftest import BF16_TOL
from oracle import decode_stack, ref

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref.available(), reason="staged reference absent")]

# 18 stacked blocks of fp32 GEMMs whose summation order differs between cuBLAS and the CPU;
# the recurrence itself is held to 1e-5 in test_gpu_field_read.py
STACK_FP32_TOL = 2e-4


def _rel(a, b):
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))


def test_prefill_and_steps_match_the_reference_full_pass():
    dev = torch.device("cuda", 0)
    batch, prefix, steps, checked = 256, 2048, 4, 3
    cpu, gpu = decode_stack.build_pair(dev)
    ids = decode_stack.token_ids(batch, prefix + steps)
    want_out, want_states = decode_stack.reference_full_pass(cpu, ids[:checked])

    got, trail = decode_stack.prefill_then_steps(gpu, ids, prefix, autocast_steps=False)
    assert got.shape == (batch, steps, decode_stack.D_MODEL)
    assert _rel(got[:checked].cpu(), want_out[:, prefix:]) < STACK_FP32_TOL
    for k in range(steps):
        for b, state in enumerate(trail[k]):
            assert _rel(state[:checked].cpu(), want_states[b][:, prefix + k]) < STACK_FP32_TOL, (k, b)

    # bf16 per-step inputs (autocast), fp32 carried state: the north-star's decode configuration
    got16, trail16 = decode_stack.prefill_then_steps(gpu, ids, prefix, autocast_steps=True)
    assert _rel(got16[:checked].cpu(), want_out[:, prefix:]) < BF16_TOL
    for b, state in enumerate(trail16[-1]):
        assert state.dtype == torch.float32
        assert _rel(state[:checked].cpu(), want_states[b][:, -1]) < BF16_TOL, b


def test_field_stack_decoder_on_the_reference_byte_lm():
    """``FieldStackDecoder`` on the reference's own field-only ``ByteLM`` (``field_triton``):
    prefill + steps reproduce the logits of the reference's full-sequence pass of the
    ``field_reference`` twin on the CPU, and greedy generation equals re-running the full model
    for every new token."""
    import fields_lm_b200
    canon = ref.load_canon()

    def lm(kind):
        torch.manual_seed(3)
        cfg = canon.ModelConfig(model=kind, dim=128, heads=4, layers=3, field_chunk=32,
                                triton_block_c=32, triton_chunk_t=64, checkpoint_blocks=False,
                                field_ff_hidden=352, transformer_ff_hidden=368)
        return canon.ByteLM(cfg).eval()

    cpu, gpu = lm("field_reference"), lm("field_triton")
    gpu.load_state_dict(cpu.state_dict(), strict=True)
    gpu = gpu.cuda()
    gen = torch.Generator().manual_seed(8)
    tokens = torch.randint(0, 256, (5, 150), generator=gen)
    with torch.no_grad():
        want = cpu(tokens)                               # [B, T, 256], full pass
    dec = fields_lm_b200.FieldStackDecoder(gpu)
    with pytest.raises(RuntimeError):
        dec.step(tokens[:, 0].cuda())
    prefix = 97
    all_logits = dec.prefill(tokens[:, :prefix].cuda(), last_only=False)
    assert _rel(all_logits.cpu(), want[:, :prefix]) < STACK_FP32_TOL
    for t in range(prefix, tokens.shape[1]):
        logits = dec.step(tokens[:, t].cuda())
        assert _rel(logits.cpu(), want[:, t]) < STACK_FP32_TOL, t
    # greedy continuation against the reference's only way of doing it: a full pass per token
    fields_lm_b200.install(gpu)
    try:
        seq = tokens[:, :40].cuda()
        out = dec.generate(seq, 6)
        for _ in range(6):
            with torch.no_grad():
                nxt = gpu(seq)[:, -1].argmax(dim=-1)
            seq = torch.cat([seq, nxt[:, None]], dim=1)
    finally:
        fields_lm_b200.uninstall(gpu)
    assert torch.equal(out, seq)
    with pytest.raises(TypeError):
        fields_lm_b200.FieldStackDecoder(torch.nn.Linear(2, 2))
