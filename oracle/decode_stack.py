"""Prefill + recurrent decode through a stack of the reference's Field blocks. TEST INFRASTRUCTURE.

The decode configuration: token ids uniform in [0, 16384) -> embedding -> 18 ``FieldBlock``s of
the staged reference (d_model 1,024, ``ff_hidden`` 2,528, seed-0 weights), a 2,048-token prefix,
then single-token steps that carry one fp32 complex state per block. The reference has no
incremental path (its inference is a full-sequence pass); because every block is causal, the
oracle for step ``k`` is the reference's own full pass over prefix + k + 1 tokens
(``field_only_v4_chunked_triton_wiki100.py:1167-1221`` with ``backend="reference"`` on the CPU):
position ``prefix + k`` of its output is what the step must return, and the state planes of
``read`` at that position are what the step must have left in the carried state.

Used by ``tests/test_gpu_decode_stack.py`` and the ``decode_step`` leg of ``bench.py``.
"""
from __future__ import annotations

from typing import List

import torch

from . import ref

VOCAB, D_MODEL, BLOCKS, FF_HIDDEN = 16_384, 1024, 18, 2528


class Stack(torch.nn.Module):
    """Embedding + ``blocks`` Field blocks of the reference, built under one seed."""

    def __init__(self, canon, backend: str, blocks: int = BLOCKS, dim: int = D_MODEL,
                 ff_hidden: int = FF_HIDDEN, vocab: int = VOCAB, seed: int = 0):
        super().__init__()
        torch.manual_seed(seed)
        self.emb = torch.nn.Embedding(vocab, dim)
        self.blocks = torch.nn.ModuleList(
            canon.FieldBlock(dim, backend, 32, 32, 64, ff_hidden) for _ in range(blocks))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        x = self.emb(ids)
        for block in self.blocks:
            x = block(x)
        return x


def token_ids(batch: int, length: int, seed: int = 4) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, VOCAB, (batch, length), generator=gen, dtype=torch.long)


@torch.no_grad()
def reference_full_pass(stack_cpu: Stack, ids: torch.Tensor):
    """The reference's full-sequence pass on the CPU: the stack's output and, per block, the
    state planes of ``read`` (the input of ``read_norm``) at every position."""
    states: List[torch.Tensor] = []
    handles = [b.mixer.read_norm.register_forward_pre_hook(
        lambda mod, args: states.append(args[0][..., :mod.weight.numel() // 2].clone()))
        for b in stack_cpu.blocks]
    try:
        out = stack_cpu(ids)
    finally:
        for h in handles:
            h.remove()
    return out, states


@torch.no_grad()
def prefill_then_steps(stack_gpu: Stack, ids: torch.Tensor, prefix: int, autocast_steps: bool,
                       rows_per_pass: int = 32):
    """This library on the GPU: a prefix pass that returns each block's end state
    (``fields_lm_b200.mixer.block_prefill``), then one ``block_step`` per new token.
    Returns (outputs of the steps ``[B, k, dim]``, carried states after every step
    ``[k][blocks][B, dim]``). ``autocast_steps``: the steps run under bf16 autocast, so the write
    projection hands the step kernel bfloat16 rows; the states stay fp32."""
    from fields_lm_b200.mixer import block_prefill, block_step
    B, total = ids.shape
    dev = next(stack_gpu.parameters()).device
    states = [torch.empty(B, stack_gpu.emb.embedding_dim, device=dev) for _ in stack_gpu.blocks]
    for lo in range(0, B, rows_per_pass):       # the prefix in slices of the batch: bounded memory
        x = stack_gpu.emb(ids[lo:lo + rows_per_pass, :prefix].to(dev))
        for block, state in zip(stack_gpu.blocks, states):
            x, s = block_prefill(block, x)
            state[lo:lo + rows_per_pass] = s
        del x
    outs, trail = [], []
    for t in range(prefix, total):
        x = stack_gpu.emb(ids[:, t].to(dev))
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast_steps):
            for block, state in zip(stack_gpu.blocks, states):
                x = block_step(block, x, state)
        outs.append(x.float())
        trail.append([s.clone() for s in states])
    return torch.stack(outs, dim=1), trail


def build_pair(device, blocks: int = BLOCKS):
    """The same seeded weights as a ``"reference"`` stack on the CPU and a ``"triton"`` stack on
    ``device`` (whose blocks this library steps through directly)."""
    canon = ref.load_canon()
    cpu = Stack(canon, "reference", blocks).eval()
    gpu = Stack(canon, "triton", blocks).eval()
    gpu.load_state_dict(cpu.state_dict(), strict=True)
    return cpu, gpu.to(device)
