"""The Field mixer's forward on the wider boundaries, as functions of the reference's own modules.

Every function takes a module with the attributes of the reference's
``IndependentVacancyField`` (``field_only_v4_chunked_triton_wiki100.py:1131-1195``:
``write_proj``, ``radius_logit``, ``theta``, ``read_norm``, ``out_proj``, ``gate_proj``,
``channels``, ``dim``) or of its ``FieldBlock`` (``:1198-1221``: ``mixer``, ``ff_norm``,
``ff``) and computes the same function of the same parameters; no parameter is added, so
checkpoints stay interchangeable. The recurrence is the CUDA operator; the three
projections, the RMS norms and the SwiGLU feed-forward stay PyTorch library calls, as in
the reference.

* :func:`fused_mixer_forward` - bfloat16 boundary, norm statistics from the recurrence
  kernel, the norm applied after the output projection, one epilogue kernel
  (``fields_lm_b200.install(model, fused_mixer=True)`` routes a model through it);
* :func:`bf16_mixer_forward` - bfloat16 boundary without that re-ordering;
* :func:`mixer_forward_with_state`, :func:`mixer_step`, :func:`block_prefill`,
  :func:`block_step` - a span that continues from a carried state, and incremental
  decoding, which the reference does not have (its inference is a full-sequence pass).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .decode import field_read_step
from .field_read import (field_read_with_state, fused_field_read_bf16,
                         fused_field_read_bf16_stats, mixer_epilogue)


def transition_parameters(radius_logit: torch.Tensor, theta: torch.Tensor):
    """``lambda = r e^{i theta}``, ``gamma = sqrt(max(1 - r^2, 1e-4))`` (reference :1169-1173)."""
    radius = torch.sigmoid(radius_logit).clamp(0.50, 0.99995).float()
    theta = theta.float()
    return (radius * torch.cos(theta), radius * torch.sin(theta),
            torch.sqrt((1.0 - radius.square()).clamp_min(1e-4)))


def fused_mixer_forward(m: nn.Module, x: torch.Tensor) -> Optional[torch.Tensor]:
    """The Field mixer's forward on the bfloat16 boundary with the norm behind the projection.

    Same function of the same parameters as reference :1167-1195:

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


def bf16_mixer_forward(m: nn.Module, x: torch.Tensor) -> Optional[torch.Tensor]:
    """The mixer with the write projection's bfloat16 output kept (no ``.float()`` widening,
    reference :1168) and the recurrence on the bfloat16 boundary, everything else as the
    reference orders it. Returns None when it does not apply (not CUDA, no bfloat16 autocast,
    channel count not a multiple of four)."""
    if not (x.is_cuda and torch.is_autocast_enabled()
            and torch.get_autocast_dtype("cuda") == torch.bfloat16 and m.channels % 4 == 0):
        return None
    raw = m.write_proj(x).contiguous()
    tr, ti, gamma = transition_parameters(m.radius_logit, m.theta)
    read = fused_field_read_bf16(raw, tr, ti, gamma)
    out = m.out_proj(m.read_norm(read))
    return x + (out * torch.sigmoid(m.gate_proj(x))).to(x.dtype)


def mixer_forward_with_state(m: nn.Module, x: torch.Tensor,
                             state_in: Optional[torch.Tensor] = None):
    """The mixer's forward for a span that continues from ``state_in [B, dim]`` (None: the zero
    state, i.e. the reference's forward); also returns the state after the span."""
    raw = m.write_proj(x).contiguous().float()
    tr, ti, gamma = transition_parameters(m.radius_logit, m.theta)
    read, state_out = field_read_with_state(raw, tr, ti, gamma, state_in)
    out = m.out_proj(m.read_norm(read))
    return x + (out * torch.sigmoid(m.gate_proj(x))).to(x.dtype), state_out


@torch.no_grad()
def mixer_step(m: nn.Module, x: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    """One new token per sequence: ``x [B, dim]``, ``state [B, dim]`` fp32 updated in place."""
    raw = m.write_proj(x).contiguous()
    if raw.dtype not in (torch.float32, torch.bfloat16):
        raw = raw.float()
    tr, ti, gamma = transition_parameters(m.radius_logit, m.theta)
    read = field_read_step(raw, tr, ti, gamma, state)
    out = m.out_proj(m.read_norm(read))
    return x + (out * torch.sigmoid(m.gate_proj(x))).to(x.dtype)


@torch.no_grad()
def block_prefill(block: nn.Module, x: torch.Tensor):
    """Full pass of a Field block over a prefix ``[B, L, dim]``; returns the output and the
    mixer's end state ``[B, dim]`` from which :func:`block_step` continues."""
    x, state = mixer_forward_with_state(block.mixer, x, None)
    return x + block.ff(block.ff_norm(x)), state


@torch.no_grad()
def block_step(block: nn.Module, x: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    """One token through a Field block: ``x [B, dim]``; ``state`` is advanced in place."""
    x = mixer_step(block.mixer, x, state)
    return x + block.ff(block.ff_norm(x))
