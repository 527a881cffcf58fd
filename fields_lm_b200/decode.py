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
