"""Incremental decoding: one recurrent step of the Field read per new token.

The reference has no incremental path (its inference is a full-sequence pass); the
recurrence is causal, so a prefix pass that returns its end state followed by
single-token steps reproduces the full pass over prefix + tokens, which is how the tests
check it. The state ``[B, 2C]`` stays fp32; inputs and outputs are fp32 or bf16.
"""
from __future__ import annotations

import torch

from . import _lib


def field_read_step(raw_row: torch.Tensor, transition_r: torch.Tensor, transition_i: torch.Tensor,
                    gamma: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    """Advances ``state`` in place by one token and returns that token's ``read`` row.

    ``raw_row`` is ``[B, 3C]`` (fp32 or bf16, CUDA, contiguous); ``state`` is ``[B, 2C]`` fp32
    and is overwritten with the new state; the result is ``[B, 4C]`` in ``raw_row``'s dtype.
    """
    if not raw_row.is_cuda:
        raise RuntimeError("Field decode step requires CUDA")
    if raw_row.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"raw_row must be float32 or bfloat16, got {raw_row.dtype}")
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise TypeError("state must be a contiguous float32 tensor")
    B, three_c = raw_row.shape
    C = three_c // 3
    if three_c % 3 or tuple(state.shape) != (B, 2 * C) or transition_r.numel() != C:
        raise ValueError((tuple(raw_row.shape), tuple(state.shape), tuple(transition_r.shape)))
    raw_row = raw_row.contiguous()
    tr = transition_r.detach().contiguous().float()
    ti = transition_i.detach().contiguous().float()
    gm = gamma.detach().contiguous().float()
    lib = _lib.load()
    with torch.cuda.device(raw_row.device):
        read = torch.empty((B, 4 * C), device=raw_row.device, dtype=raw_row.dtype)
        fn = lib.fields_read_step if raw_row.dtype == torch.float32 else lib.fields_read_step_bf16
        rc = fn(raw_row.data_ptr(), tr.data_ptr(), ti.data_ptr(), gm.data_ptr(), state.data_ptr(),
                read.data_ptr(), B, C, torch.cuda.current_stream(raw_row.device).cuda_stream)
    _lib.check(rc, "fields_read_step")
    return read


class FieldStackDecoder:
    """Stateful prefill -> decode for a language model made of the reference's Field blocks.

    Works on any module shaped like the reference's field-only ``ByteLM``
    (``field_only_v4_chunked_triton_wiki100.py:1306-1344`` with ``model="field_triton"``): an
    embedding ``emb``, a list ``blocks`` of ``FieldBlock``s, ``final_norm`` and ``lm_head``. The
    reference itself can only run the whole sequence again for every new token; here
    :meth:`prefill` runs the prompt once and keeps one fp32 state ``[B, dim]`` per block, and
    :meth:`step` advances all of them by one token. The hybrid ``FieldsForCausalLM`` is not
    covered: its refresh-attention and Mamba-2 layers would need caches of their own.
    """

    def __init__(self, model: torch.nn.Module):
        for name in ("emb", "blocks", "final_norm", "lm_head"):
            if not hasattr(model, name):
                raise TypeError(f"model has no `{name}`: not a field-only language model")
        for block in model.blocks:
            if type(block).__name__ != "FieldBlock":
                raise TypeError(f"block of type {type(block).__name__}: only FieldBlock can be "
                                "stepped")
        self.model = model
        self.states = None

    def reset(self) -> None:
        self.states = None

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, last_only: bool = True) -> torch.Tensor:
        """Runs the prompt ``tokens [B, T]`` and stores the blocks' end states. Returns the
        logits of the last position ``[B, V]``, or of every position with ``last_only=False``."""
        from .mixer import block_prefill
        x = self.model.emb(tokens)
        states = []
        for block in self.model.blocks:
            x, state = block_prefill(block, x)
            states.append(state)
        self.states = states
        if last_only:
            x = x[:, -1]
        return self.model.lm_head(self.model.final_norm(x))

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """One new token per sequence, ``tokens [B]``; returns its logits ``[B, V]``."""
        from .mixer import block_step
        if self.states is None:
            raise RuntimeError("call prefill() before step()")
        x = self.model.emb(tokens)
        for block, state in zip(self.model.blocks, self.states):
            x = block_step(block, x, state)
        return self.model.lm_head(self.model.final_norm(x))

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy continuation of ``prompt [B, T]`` by ``new_tokens`` tokens."""
        logits = self.prefill(prompt)
        out = [prompt]
        for _ in range(new_tokens):
            nxt = logits.argmax(dim=-1)
            out.append(nxt[:, None])
            logits = self.step(nxt)
        return torch.cat(out, dim=1)
