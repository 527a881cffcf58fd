"""``fused_field_read`` on the CUDA library: the drop-in for the reference's operator.

Mirrors ``_ChunkedFieldReadFunction`` / ``fused_field_read`` of the reference
(``field_only_v4_chunked_triton_wiki100.py:912-1123``): same arguments, same
output layout, same gradients, same argument errors. ``block_c`` and ``chunk_t``
are launch hints of the reference's Triton kernels and are accepted and ignored.

``field_read_with_state`` is the same operator with an incoming state and the
outgoing state returned - what the sequence-sharded forward and incremental
decoding need; the reference always starts from the zero state.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

_FWD, _BWD = 0, 1


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _workspace(B: int, L: int, C: int, which: int, device) -> Tuple[torch.Tensor, int]:
    nbytes = _lib.load().fields_read_workspace_bytes(B, L, C, which)
    # the caching allocator hands out 512-byte aligned blocks
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device), nbytes


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class FieldReadFunction(torch.autograd.Function):
    """read, state_out = F(raw, tr, ti, gamma, state_in[, lean]).

    With ``lean`` the function does not keep ``read`` for its backward pass but only every
    eighth state row (1/16 of it); the backward kernel recomputes the states in between.
    """

    @staticmethod
    def forward(ctx, raw, transition_r, transition_i, gamma, state_in, lean=False):
        if not raw.is_cuda:
            raise RuntimeError("Chunked Field kernel requires CUDA")
        if raw.dtype != torch.float32:
            raise TypeError(f"raw must be float32, got {raw.dtype}")
        if raw.dim() != 3:
            raise ValueError(tuple(raw.shape))
        raw = raw.contiguous()
        tr = transition_r.contiguous().float()
        ti = transition_i.contiguous().float()
        gm = gamma.contiguous().float()
        B, L, three_c = raw.shape
        if three_c % 3:
            raise ValueError(tuple(raw.shape))
        C = three_c // 3
        if tr.numel() != C or ti.numel() != C or gm.numel() != C:
            raise ValueError((tuple(raw.shape), tuple(tr.shape)))
        if state_in is not None:
            if tuple(state_in.shape) != (B, 2 * C):
                raise ValueError((tuple(raw.shape), tuple(state_in.shape)))
            state_in = state_in.contiguous().float()
        lib = _lib.load()
        with torch.cuda.device(raw.device):
            read = torch.empty((B, L, 4 * C), device=raw.device, dtype=torch.float32)
            state_out = torch.empty((B, 2 * C), device=raw.device, dtype=torch.float32)
            ws, nbytes = _workspace(B, L, C, _FWD, raw.device)
            rc = lib.fields_read_forward(_ptr(raw), _ptr(tr), _ptr(ti), _ptr(gm), _ptr(state_in),
                                         _ptr(read), _ptr(state_out), _ptr(ws), nbytes,
                                         B, L, C, _stream(raw.device))
        _lib.check(rc, "fields_read_forward")
        ctx.set_materialize_grads(False)
        ctx.lean = bool(lean) and C % 4 == 0
        if ctx.lean:
            rows = lib.fields_read_state_rows(L)
            kept = read[:, 7::8, :2 * C][:, :rows].contiguous()
        else:
            kept = read
        ctx.save_for_backward(raw, tr, ti, gm, kept, state_in)
        ctx.dims = (B, L, C)
        return read, state_out

    @staticmethod
    def backward(ctx, grad_read, grad_state_out):
        raw, tr, ti, gm, read, state_in = ctx.saved_tensors
        B, L, C = ctx.dims
        lib = _lib.load()
        with torch.cuda.device(raw.device):
            if grad_read is None:
                grad_read = torch.zeros((B, L, 4 * C), device=raw.device, dtype=torch.float32)
            grad_read = grad_read.contiguous().float()
            if grad_state_out is not None:
                grad_state_out = grad_state_out.contiguous().float()
            grad_raw = torch.empty_like(raw)
            g_par = torch.empty((3, C), device=raw.device, dtype=torch.float32)
            g_sin = (torch.empty((B, 2 * C), device=raw.device, dtype=torch.float32)
                     if state_in is not None and ctx.needs_input_grad[4] else None)
            ws, nbytes = _workspace(B, L, C, _BWD, raw.device)
            # lean: `read` holds the kept state rows (possibly none for L <= 8)
            entry = lib.fields_read_backward_from_states if ctx.lean else lib.fields_read_backward
            rc = entry(
                _ptr(raw), _ptr(tr), _ptr(ti), _ptr(gm), _ptr(state_in),
                _ptr(read) if read.numel() else None,
                _ptr(grad_read), _ptr(grad_state_out), _ptr(grad_raw), _ptr(g_par[0]),
                _ptr(g_par[1]), _ptr(g_par[2]), _ptr(g_sin), _ptr(ws), nbytes, B, L, C,
                _stream(raw.device))
        _lib.check(rc, "fields_read_backward")
        return grad_raw, g_par[0], g_par[1], g_par[2], g_sin, None


class FieldReadBf16Function(torch.autograd.Function):
    """read = F(raw, tr, ti, gamma) with bfloat16 raw / read / gradients and an fp32 state."""

    @staticmethod
    def forward(ctx, raw, transition_r, transition_i, gamma):
        if not raw.is_cuda:
            raise RuntimeError("Chunked Field kernel requires CUDA")
        if raw.dtype != torch.bfloat16:
            raise TypeError(f"raw must be bfloat16, got {raw.dtype}")
        if raw.dim() != 3 or raw.shape[2] % 3:
            raise ValueError(tuple(raw.shape))
        raw = raw.contiguous()
        tr = transition_r.contiguous().float()
        ti = transition_i.contiguous().float()
        gm = gamma.contiguous().float()
        B, L, three_c = raw.shape
        C = three_c // 3
        if tr.numel() != C or ti.numel() != C or gm.numel() != C:
            raise ValueError((tuple(raw.shape), tuple(tr.shape)))
        lib = _lib.load()
        with torch.cuda.device(raw.device):
            read = torch.empty((B, L, 4 * C), device=raw.device, dtype=torch.bfloat16)
            ws, nbytes = _workspace(B, L, C, _FWD, raw.device)
            rc = lib.fields_read_forward_bf16(_ptr(raw), _ptr(tr), _ptr(ti), _ptr(gm), None,
                                              _ptr(read), None, _ptr(ws), nbytes, B, L, C,
                                              _stream(raw.device))
        _lib.check(rc, "fields_read_forward_bf16")
        ctx.save_for_backward(raw, tr, ti, gm, read)
        ctx.dims = (B, L, C)
        return read

    @staticmethod
    def backward(ctx, grad_read):
        raw, tr, ti, gm, read = ctx.saved_tensors
        B, L, C = ctx.dims
        lib = _lib.load()
        with torch.cuda.device(raw.device):
            grad_read = grad_read.contiguous().to(torch.bfloat16)
            grad_raw = torch.empty_like(raw)
            g_par = torch.empty((3, C), device=raw.device, dtype=torch.float32)
            ws, nbytes = _workspace(B, L, C, _BWD, raw.device)
            rc = lib.fields_read_backward_bf16(
                _ptr(raw), _ptr(tr), _ptr(ti), _ptr(gm), None, _ptr(read), _ptr(grad_read), None,
                _ptr(grad_raw), _ptr(g_par[0]), _ptr(g_par[1]), _ptr(g_par[2]), None, _ptr(ws),
                nbytes, B, L, C, _stream(raw.device))
        _lib.check(rc, "fields_read_backward_bf16")
        return grad_raw, g_par[0], g_par[1], g_par[2]


class FieldReadBf16StatsFunction(torch.autograd.Function):
    """read, sumsq = F(raw, tr, ti, gamma): the bfloat16 operator plus, per token, the sum of the
    squares of its 4C outputs (``sumsq [B, L]`` fp32, from the fp32 values before rounding)."""

    @staticmethod
    def forward(ctx, raw, transition_r, transition_i, gamma):
        if not raw.is_cuda:
            raise RuntimeError("Chunked Field kernel requires CUDA")
        if raw.dtype != torch.bfloat16:
            raise TypeError(f"raw must be bfloat16, got {raw.dtype}")
        if raw.dim() != 3 or raw.shape[2] % 3 or raw.shape[0] == 0 or raw.shape[1] == 0:
            raise ValueError(tuple(raw.shape))
        raw = raw.contiguous()
        tr = transition_r.contiguous().float()
        ti = transition_i.contiguous().float()
        gm = gamma.contiguous().float()
        B, L, three_c = raw.shape
        C = three_c // 3
        if tr.numel() != C or ti.numel() != C or gm.numel() != C:
            raise ValueError((tuple(raw.shape), tuple(tr.shape)))
        lib = _lib.load()
        with torch.cuda.device(raw.device):
            read = torch.empty((B, L, 4 * C), device=raw.device, dtype=torch.bfloat16)
            groups = torch.empty((B, L, (C + 127) // 128), device=raw.device, dtype=torch.float32)
            ws, nbytes = _workspace(B, L, C, _FWD, raw.device)
            rc = lib.fields_read_forward_bf16_stats(_ptr(raw), _ptr(tr), _ptr(ti), _ptr(gm), None,
                                                    _ptr(read), _ptr(groups), None, _ptr(ws), nbytes,
                                                    B, L, C, _stream(raw.device))
            _lib.check(rc, "fields_read_forward_bf16_stats")
            sumsq = groups.sum(dim=-1)
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(raw, tr, ti, gm, read)
        ctx.dims = (B, L, C)
        return read, sumsq

    @staticmethod
    def backward(ctx, grad_read, grad_sumsq):
        raw, tr, ti, gm, read = ctx.saved_tensors
        B, L, C = ctx.dims
        lib = _lib.load()
        with torch.cuda.device(raw.device):
            # d sumsq / d read = 2 read: folded into the gradient the recurrence receives
            if grad_sumsq is not None:
                if grad_read is not None:
                    grad_read = grad_read.contiguous().to(torch.bfloat16)
                total = torch.empty_like(read)
                rc = lib.fields_read_norm_grad_combine(_ptr(grad_read), _ptr(read),
                                                       _ptr(grad_sumsq.contiguous().float()),
                                                       _ptr(total), B * L, 4 * C,
                                                       _stream(raw.device))
                _lib.check(rc, "fields_read_norm_grad_combine")
            elif grad_read is not None:
                total = grad_read.contiguous().to(torch.bfloat16)
            else:
                total = torch.zeros_like(read)
            grad_raw = torch.empty_like(raw)
            g_par = torch.empty((3, C), device=raw.device, dtype=torch.float32)
            ws, nbytes = _workspace(B, L, C, _BWD, raw.device)
            rc = lib.fields_read_backward_bf16(
                _ptr(raw), _ptr(tr), _ptr(ti), _ptr(gm), None, _ptr(read), _ptr(total), None,
                _ptr(grad_raw), _ptr(g_par[0]), _ptr(g_par[1]), _ptr(g_par[2]), None, _ptr(ws),
                nbytes, B, L, C, _stream(raw.device))
        _lib.check(rc, "fields_read_backward_bf16")
        return grad_raw, g_par[0], g_par[1], g_par[2]


def fused_field_read_bf16_stats(raw: torch.Tensor, transition_r: torch.Tensor,
                                transition_i: torch.Tensor, gamma: torch.Tensor):
    """``fused_field_read_bf16`` that also returns ``sumsq [B, L]`` (fp32): the sum of squares of
    each token's 4C outputs, which is all an RMS norm over ``read`` needs from it. Both outputs
    are differentiable."""
    return FieldReadBf16StatsFunction.apply(raw, transition_r, transition_i, gamma)


class MixerEpilogueFunction(torch.autograd.Function):
    """y = x + (acc * rsqrt(sumsq / features + eps) + bias) * sigmoid(gate + gate_bias), one
    kernel each way."""

    @staticmethod
    def forward(ctx, x, acc, gate, sumsq, bias, gate_bias, eps, features):
        lib = _lib.load()
        D = x.shape[-1]
        x, acc, gate = x.contiguous(), acc.contiguous(), gate.contiguous()
        sumsq, bias = sumsq.contiguous().float(), bias.contiguous().float()
        if gate_bias is not None:
            gate_bias = gate_bias.contiguous().float()
        N = x.numel() // D
        y = torch.empty_like(x)
        with torch.cuda.device(x.device):
            rc = lib.fields_mixer_epilogue_forward(_ptr(x), _ptr(acc), _ptr(gate), _ptr(sumsq),
                                                   _ptr(bias), _ptr(gate_bias), _ptr(y), float(eps),
                                                   int(features), N, D, _stream(x.device))
        _lib.check(rc, "fields_mixer_epilogue_forward")
        ctx.save_for_backward(acc, gate, sumsq, bias, gate_bias)
        ctx.consts = (float(eps), int(features), N, D)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        acc, gate, sumsq, bias, gate_bias = ctx.saved_tensors
        eps, features, N, D = ctx.consts
        lib = _lib.load()
        grad_y = grad_y.contiguous().float()
        with torch.cuda.device(grad_y.device):
            grad_acc, grad_gate = torch.empty_like(acc), torch.empty_like(gate)
            grad_sumsq = torch.empty_like(sumsq)
            rows = lib.fields_mixer_epilogue_bias_rows(N)
            bias_rows = torch.empty((2 if gate_bias is not None else 1, rows, D),
                                    device=grad_y.device, dtype=torch.float32)
            rc = lib.fields_mixer_epilogue_backward(
                _ptr(grad_y), _ptr(acc), _ptr(gate), _ptr(sumsq), _ptr(bias), _ptr(gate_bias),
                _ptr(grad_acc), _ptr(grad_gate), _ptr(grad_sumsq), _ptr(bias_rows[0]),
                _ptr(bias_rows[1]) if gate_bias is not None else None, eps, features, N, D,
                _stream(grad_y.device))
            _lib.check(rc, "fields_mixer_epilogue_backward")
            sums = bias_rows.sum(dim=1)
        return (grad_y, grad_acc, grad_gate, grad_sumsq, sums[0],
                sums[1] if gate_bias is not None else None, None, None)


def mixer_epilogue(x: torch.Tensor, acc: torch.Tensor, gate: torch.Tensor, sumsq: torch.Tensor,
                   bias: torch.Tensor, eps: float, features: int,
                   gate_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x + (acc * rsqrt(sumsq / features + eps) + bias) * sigmoid(gate + gate_bias)`` in one CUDA
    kernel (and one for all gradients): ``x [..., D]`` fp32, ``acc`` and ``gate`` ``[..., D]``
    bfloat16, ``sumsq [...]`` fp32 (per token), ``bias``, ``gate_bias`` ``[D]`` (the latter
    optional); ``D`` a multiple of 4, at most 4096."""
    if x.dtype != torch.float32 or acc.dtype != torch.bfloat16 or gate.dtype != torch.bfloat16:
        raise TypeError((x.dtype, acc.dtype, gate.dtype))
    return MixerEpilogueFunction.apply(x, acc, gate, sumsq, bias, gate_bias, eps, features)


def fused_field_read_bf16(raw: torch.Tensor, transition_r: torch.Tensor,
                          transition_i: torch.Tensor, gamma: torch.Tensor) -> torch.Tensor:
    """The operator on a bfloat16 boundary: ``raw [B, L, 3C]`` bf16 in, ``read [B, L, 4C]`` bf16
    out, fp32 state inside. For mixers that keep the write projection's bf16 output."""
    return FieldReadBf16Function.apply(raw, transition_r, transition_i, gamma)


def fused_field_read(raw: torch.Tensor, transition_r: torch.Tensor, transition_i: torch.Tensor,
                     gamma: torch.Tensor, block_c: int = 32, chunk_t: int = 64) -> torch.Tensor:
    """Drop-in for the reference's ``fused_field_read``; returns ``read [B, L, 4C]`` fp32."""
    read, _ = FieldReadFunction.apply(raw, transition_r, transition_i, gamma, None)
    return read


def field_read_with_state(raw, transition_r, transition_i, gamma,
                          state_in: Optional[torch.Tensor] = None, lean: bool = False):
    """Same operator with a carried state: returns ``(read, state_out [B, 2C])``.

    ``lean=True`` keeps only every eighth state row for the backward pass instead of ``read``
    (the kernel recomputes the rest; about 7 % slower backward, 8 KB per token less saved by
    this operator). It pays when the consumer of ``read`` does not keep it either.
    """
    return FieldReadFunction.apply(raw, transition_r, transition_i, gamma, state_in, lean)
