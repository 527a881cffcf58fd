"""``hierarchical_scan`` for real fp32 CUDA tensors on the CUDA library.

The reference's scan primitive ``hierarchical_scan(a, b, block=32)``
(``field_only_v4_chunked_triton_wiki100.py:347-391``) has a second call site besides the
Field read: the softpatch ``FastBoundaryStateMixer`` runs it on a rank-64 real state with one
decay per token expanded over the channels
(``official_source/field_hybrid_speed_optimization_v6.py:333-335``). ``linear_scan`` is that
call on this library's ``fields_scan_forward`` / ``fields_scan_backward``: same arguments, same
output ``[B, L, C]``, gradients for ``a`` and ``b``, the same ``ValueError`` for ``block``
outside ``[1, 64]`` (``block`` itself is a blocking hint of the reference and does not change
the result).

``scan_entry(original)`` builds the function that :func:`fields_lm_b200.install` puts in place
of the module global: real fp32 CUDA inputs run here, everything else (the complex CPU call of
``reference_field_read``) goes to the reference's own function untouched.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import _lib
from .field_read import _ptr, _stream


def _a_layout(a: torch.Tensor, B: int, L: int, C: int):
    """``a`` as the library reads it: a dense tensor, or one value per (b, t) broadcast over the
    channels (the expanded view the softpatch mixer passes). Returns (tensor, batch, step, chan)."""
    if C > 1 and a.stride(2) == 0:
        per_token = a[:, :, 0].contiguous()
        return per_token, L, 1, 0
    a = a.contiguous()
    return a, L * C, C, 1


class LinearScanFunction(torch.autograd.Function):
    """states, state_out = F(a, b, state_in): ``s_t = a_t s_{t-1} + b_t`` along dim 1."""

    @staticmethod
    def forward(ctx, a, b, state_in):
        B, L, C = b.shape
        b = b.contiguous()
        a_mem, a_batch, a_step, a_chan = _a_layout(a, B, L, C)
        if state_in is not None:
            if tuple(state_in.shape) != (B, C):
                raise ValueError((tuple(b.shape), tuple(state_in.shape)))
            state_in = state_in.contiguous().float()
        lib = _lib.load()
        with torch.cuda.device(b.device):
            states = torch.empty_like(b)
            state_out = torch.empty((B, C), device=b.device, dtype=torch.float32)
            nbytes = lib.fields_scan_workspace_bytes(B, L, C)
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=b.device)
            rc = lib.fields_scan_forward(_ptr(a_mem), a_batch, a_step, a_chan, _ptr(b),
                                         _ptr(state_in), _ptr(states), _ptr(state_out), _ptr(ws),
                                         nbytes, B, L, C, _stream(b.device))
        _lib.check(rc, "fields_scan_forward")
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(a_mem, states, state_in)
        ctx.layout = (a_batch, a_step, a_chan)
        ctx.dims = (B, L, C)
        return states, state_out

    @staticmethod
    def backward(ctx, grad_states, grad_state_out):
        a_mem, states, state_in = ctx.saved_tensors
        a_batch, a_step, a_chan = ctx.layout
        B, L, C = ctx.dims
        lib = _lib.load()
        dev = states.device
        with torch.cuda.device(dev):
            if grad_states is None:
                grad_states = torch.zeros_like(states)
            grad_states = grad_states.contiguous().float()
            if grad_state_out is not None:
                grad_state_out = grad_state_out.contiguous().float()
            grad_a = torch.empty_like(states)
            grad_b = torch.empty_like(states)
            g_sin = (torch.empty((B, C), device=dev, dtype=torch.float32)
                     if state_in is not None and ctx.needs_input_grad[2] else None)
            nbytes = lib.fields_scan_workspace_bytes(B, L, C)
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
            rc = lib.fields_scan_backward(_ptr(a_mem), a_batch, a_step, a_chan, _ptr(states),
                                          _ptr(state_in), _ptr(grad_states), _ptr(grad_state_out),
                                          _ptr(grad_a), _ptr(grad_b), _ptr(g_sin), _ptr(ws), nbytes,
                                          B, L, C, _stream(dev))
        _lib.check(rc, "fields_scan_backward")
        # dense gradient of `a`; for an expanded `a` autograd sums it over the broadcast channels
        return (grad_a if ctx.needs_input_grad[0] else None), grad_b, g_sin


def _check(a: torch.Tensor, b: torch.Tensor, block: int) -> None:
    if block < 1 or block > 64:
        raise ValueError("field_chunk must be in [1, 64]")
    if not b.is_cuda or not a.is_cuda:
        raise RuntimeError("linear_scan requires CUDA tensors")
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise TypeError(f"a and b must be float32, got {a.dtype} and {b.dtype}")
    if a.dim() != 3 or a.shape != b.shape:
        raise ValueError((tuple(a.shape), tuple(b.shape)))


def linear_scan(a: torch.Tensor, b: torch.Tensor, block: int = 32) -> torch.Tensor:
    """The reference's ``hierarchical_scan(a, b, block)`` for real fp32 CUDA tensors."""
    _check(a, b, block)
    return LinearScanFunction.apply(a, b, None)[0]


def linear_scan_with_state(a: torch.Tensor, b: torch.Tensor,
                           state_in: Optional[torch.Tensor] = None):
    """The same scan from an incoming state ``[B, C]``; returns (states, state after the last
    step). An extension: the reference always starts from zero."""
    _check(a, b, 32)
    return LinearScanFunction.apply(a, b, state_in)


def scan_entry(original: Callable) -> Callable:
    """The replacement for a module's ``hierarchical_scan`` global: real fp32 CUDA calls run on
    this library, every other call (complex tensors, CPU tensors, other dtypes) goes to
    ``original`` exactly as before."""

    def hierarchical_scan(a, b, block: int = 32):
        if (torch.is_tensor(a) and torch.is_tensor(b) and a.is_cuda and b.is_cuda
                and a.dtype == torch.float32 and b.dtype == torch.float32
                and a.dim() == 3 and a.shape == b.shape):
            return linear_scan(a, b, block)
        return original(a, b, block)

    hierarchical_scan.__wrapped__ = original
    return hierarchical_scan
