"""Host-side mirror of the reference's Field mixer and Field block.

Same parameters, names, initialisation order and arithmetic as
``IndependentVacancyField`` and ``FieldBlock``
(``field_only_v4_chunked_triton_wiki100.py:1131-1221``), so a ``state_dict`` moves
between the two unchanged and a block built under the same seed holds the same
weights. The recurrence is the CUDA operator; the three projections, the RMS
norms and the SwiGLU feed-forward stay PyTorch library calls, as in the
reference. It exists so that the block-level call site can be exercised where the
reference checkout is not present; with the reference at hand, use
``fields_lm_b200.install`` on the reference's own modules instead.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .decode import field_read_step
from .field_read import (field_read_with_state, fused_field_read, fused_field_read_bf16,
                         fused_field_read_bf16_stats, mixer_epilogue)


class RMSNorm(nn.Module):
    """fp32 RMS norm with a learned scale (reference :300-309)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        return (xf * inv * self.weight.float()).to(x.dtype)


class PackedSwiGLU(nn.Module):
    """SwiGLU feed-forward with gate and value in one projection (reference :312-325)."""

    def __init__(self, dim: int, hidden: Optional[int] = None):
        super().__init__()
        self.hidden = int(hidden) if hidden is not None else ((int(8 * dim / 3) + 63) // 64) * 64
        self.w12 = nn.Linear(dim, 2 * self.hidden, bias=False)
        self.w3 = nn.Linear(self.hidden, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gate, value = self.w12(x).chunk(2, dim=-1)
        return self.w3(F.silu(gate) * value)


def transition_parameters(radius_logit: torch.Tensor, theta: torch.Tensor):
    """``lambda = r e^{i theta}``, ``gamma = sqrt(max(1 - r^2, 1e-4))`` (reference :1169-1173)."""
    radius = torch.sigmoid(radius_logit).clamp(0.50, 0.99995).float()
    theta = theta.float()
    return (radius * torch.cos(theta), radius * torch.sin(theta),
            torch.sqrt((1.0 - radius.square()).clamp_min(1e-4)))


def fused_mixer_forward(m: nn.Module, x: torch.Tensor) -> Optional[torch.Tensor]:
    """The Field mixer's forward on the bfloat16 boundary with the norm behind the projection.

    Works on any module with the reference mixer's attributes (``write_proj``, ``radius_logit``,
    ``theta``, ``read_norm``, ``out_proj``, ``gate_proj``, ``channels``, ``dim``): the mirror below
    and the reference's own ``IndependentVacancyField`` (``fields_lm_b200.install(...,
    fused_mixer=True)``). Same function of the same parameters as reference :1167-1195:

        out_proj(read_norm(read)) = rstd * (read @ (W diag(w))^T) + b

    with ``rstd`` from the sums of squares that the recurrence kernel returns, so ``read`` goes
    from the recurrence to the GEMM in bfloat16 with no reduction pass and no normalised copy;
    scale, both biases, sigmoid gate and residual are one kernel. Returns None when it does not
    apply (not CUDA, no bfloat16 autocast, fp32 input expected, channel count not a multiple of
    four): the caller then runs the ordinary forward.
    """
    if not (x.is_cuda and x.dtype == torch.float32 and torch.is_autocast_enabled()
            and torch.get_autocast_dtype("cuda") == torch.bfloat16
            and m.channels % 4 == 0 and m.dim % 4 == 0 and m.dim <= 4096):
        return None
    x_in = x.to(torch.bfloat16)  # both projections of x take the same copy
    raw = m.write_proj(x_in).contiguous()
    tr, ti, gamma = transition_parameters(m.radius_logit, m.theta)
    read, sumsq = fused_field_read_bf16_stats(raw, tr, ti, gamma)
    w_eff = m.out_proj.weight.float() * m.read_norm.weight.float().unsqueeze(0)
    acc = F.linear(read, w_eff.to(read.dtype))
    gate = F.linear(x_in, m.gate_proj.weight)
    # the gate projection's bias is added, and its gradient summed, inside the epilogue kernels
    return mixer_epilogue(x, acc, gate, sumsq, m.out_proj.bias, m.read_norm.eps, read.shape[-1],
                          gate_bias=m.gate_proj.bias)


class IndependentVacancyField(nn.Module):
    """Field mixer: write projection -> recurrence -> norm, output projection, gate, residual."""

    def __init__(self, dim: int, backend: str = "triton", field_chunk: int = 32,
                 triton_block_c: int = 32, triton_chunk_t: int = 64):
        super().__init__()
        if dim % 2:
            raise ValueError("Field dim must be even")
        if backend not in ("reference", "triton"):
            raise ValueError(backend)
        self.dim = dim
        self.channels = dim // 2
        self.backend = backend
        self.field_chunk = int(field_chunk)
        self.triton_block_c = int(triton_block_c)
        self.triton_chunk_t = int(triton_chunk_t)
        self.write_proj = nn.Linear(dim, dim + self.channels)
        ring = torch.linspace(0.85, 0.999, self.channels)
        self.radius_logit = nn.Parameter(torch.log(ring / (1.0 - ring)))
        self.theta = nn.Parameter(torch.linspace(0.03, math.pi * 0.97, self.channels))
        self.read_norm = RMSNorm(2 * dim)
        self.out_proj = nn.Linear(2 * dim, dim)
        self.gate_proj = nn.Linear(dim, dim)
        # Not a constructor argument (the signature mirrors the reference's): set to True to keep
        # the write projection's bf16 output under autocast and run the recurrence on a bfloat16
        # boundary (fp32 state) instead of widening raw to fp32 first.
        self.bf16_io = False
        # With bf16_io: run fused_mixer_forward (norm statistics from the recurrence kernel, norm
        # applied after the output projection, one epilogue kernel) whenever it applies.
        self.fused_norm = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.bf16_io and self.fused_norm:
            y = fused_mixer_forward(self, x)
            if y is not None:
                return y
        raw = self.write_proj(x).contiguous()
        if self.bf16_io and raw.dtype == torch.bfloat16:
            tr, ti, gamma = transition_parameters(self.radius_logit, self.theta)
            read = fused_field_read_bf16(raw, tr, ti, gamma)
            out = self.out_proj(self.read_norm(read))
            return x + (out * torch.sigmoid(self.gate_proj(x))).to(x.dtype)
        raw = raw.float()
        tr, ti, gamma = transition_parameters(self.radius_logit, self.theta)
        read = fused_field_read(raw, tr, ti, gamma, self.triton_block_c, self.triton_chunk_t)
        out = self.out_proj(self.read_norm(read))
        return x + (out * torch.sigmoid(self.gate_proj(x))).to(x.dtype)

    def forward_with_state(self, x: torch.Tensor, state_in: Optional[torch.Tensor] = None):
        """Same as ``forward`` for a span that continues from ``state_in``; also returns the end state."""
        raw = self.write_proj(x).contiguous().float()
        tr, ti, gamma = transition_parameters(self.radius_logit, self.theta)
        read, state_out = field_read_with_state(raw, tr, ti, gamma, state_in)
        out = self.out_proj(self.read_norm(read))
        return x + (out * torch.sigmoid(self.gate_proj(x))).to(x.dtype), state_out


    @torch.no_grad()
    def step(self, x: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        """One new token per sequence: ``x [B, dim]``, ``state [B, dim]`` fp32 updated in place."""
        raw = self.write_proj(x).contiguous()
        if raw.dtype not in (torch.float32, torch.bfloat16):
            raw = raw.float()
        tr, ti, gamma = transition_parameters(self.radius_logit, self.theta)
        read = field_read_step(raw, tr, ti, gamma, state)
        out = self.out_proj(self.read_norm(read))
        return x + (out * torch.sigmoid(self.gate_proj(x))).to(x.dtype)


class FieldBlock(nn.Module):
    """Field mixer followed by a pre-norm SwiGLU feed-forward (reference :1198-1221)."""

    def __init__(self, dim: int, backend: str = "triton", field_chunk: int = 32,
                 triton_block_c: int = 32, triton_chunk_t: int = 64, ff_hidden: Optional[int] = None):
        super().__init__()
        self.mixer = IndependentVacancyField(dim, backend, field_chunk, triton_block_c,
                                             triton_chunk_t)
        self.ff_norm = RMSNorm(dim)
        self.ff = PackedSwiGLU(dim, hidden=ff_hidden)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.mixer(x)
        return x + self.ff(self.ff_norm(x))

    @torch.no_grad()
    def prefill(self, x: torch.Tensor):
        """Full pass over a prefix ``[B, L, dim]``; returns the output and the mixer's end state."""
        x, state = self.mixer.forward_with_state(x, None)
        return x + self.ff(self.ff_norm(x)), state

    @torch.no_grad()
    def step(self, x: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        x = self.mixer.step(x, state)
        return x + self.ff(self.ff_norm(x))
