"""PyTorch CPU port of the reference's Field read (test infrastructure only).

Same arithmetic and the same scan shape as the reference's complex64 path, so
that timing it on the host cores stands for the reference's own CPU speed:

* ``doubling_scan``   — log-step inclusive scan of ``s_t = a_t s_{t-1} + b_t``
  (``field_only_v4_chunked_triton_wiki100.py:333-344``).
* ``blocked_scan``    — scan inside blocks of ``block`` steps, scan of the
  block summaries, recombination (``:347-389``); no prefix division.
* ``field_read``      — gates, complex coefficients, scan, displaced readout
  (``:392-416``).
* ``transition_parameters`` — ``radius_logit, theta -> lambda_r, lambda_i,
  gamma`` (``:1169-1173``).

Backward is PyTorch autograd through these complex ops, as in the reference.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

VAC_MAX = 0.90  # field_only_v4_chunked_triton_wiki100.py:68


def _shift_time(x: torch.Tensor, k: int, fill: float) -> torch.Tensor:
    """x delayed by k steps along dim 1, the first k steps filled with ``fill``."""
    head = torch.full_like(x[:, :k], fill)
    return torch.cat((head, x[:, : x.shape[1] - k]), dim=1)


def doubling_scan(a: torch.Tensor, b: torch.Tensor):
    """Inclusive scan along dim 1; returns (prefix product of a, states from s_-1 = 0)."""
    a = a.clone()
    b = b.clone()
    k = 1
    n = a.shape[1]
    while k < n:
        b = a * _shift_time(b, k, 0.0) + b
        a = a * _shift_time(a, k, 1.0)
        k *= 2
    return a, b


def blocked_scan(a: torch.Tensor, b: torch.Tensor, block: int = 32) -> torch.Tensor:
    if not 1 <= block <= 64:
        raise ValueError("field_chunk must be in [1, 64]")
    B, L, C = a.shape
    pad = (-L) % block
    if pad:
        a = torch.cat((a, a.new_ones(B, pad, C)), dim=1)
        b = torch.cat((b, b.new_zeros(B, pad, C)), dim=1)
    G = a.shape[1] // block
    la, lb = doubling_scan(a.reshape(B * G, block, C), b.reshape(B * G, block, C))
    la = la.reshape(B, G, block, C)
    lb = lb.reshape(B, G, block, C)
    _, ends = doubling_scan(la[:, :, -1], lb[:, :, -1])
    carry = _shift_time(ends, 1, 0.0)
    states = la * carry[:, :, None, :] + lb
    return states.reshape(B, G * block, C)[:, :L]


def field_read(raw: torch.Tensor, tr: torch.Tensor, ti: torch.Tensor,
               gamma: torch.Tensor, field_chunk: int = 32) -> torch.Tensor:
    C = tr.numel()
    zr, zi, zv = raw[..., :C], raw[..., C:2 * C], raw[..., 2 * C:]
    inj = torch.complex(torch.tanh(zr), torch.tanh(zi))
    vac = (torch.sigmoid(zv) * VAC_MAX).to(torch.complex64)
    lam = torch.complex(tr, ti)
    a = (1.0 - vac) * lam
    b = gamma.to(torch.complex64) * vac * inj
    s = blocked_scan(a, b, field_chunk)
    disp = vac * (lam * _shift_time(s, 1, 0.0))
    return torch.cat((s.real, s.imag, disp.real, disp.imag), dim=-1)


def transition_parameters(radius_logit: torch.Tensor, theta: torch.Tensor):
    radius = torch.sigmoid(radius_logit).clamp(0.50, 0.99995).float()
    theta = theta.float()
    tr = radius * torch.cos(theta)
    ti = radius * torch.sin(theta)
    gamma = torch.sqrt((1.0 - radius.square()).clamp_min(1e-4))
    return tr, ti, gamma


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm in fp32 (field_only_v4_chunked_triton_wiki100.py:300-309)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def mixer_forward(params: dict, x: torch.Tensor, field_chunk: int = 32) -> torch.Tensor:
    """Field mixer on CPU from a state-dict of the mixer's parameters (:1167-1195)."""
    raw = F.linear(x, params["write_proj.weight"], params["write_proj.bias"]).contiguous().float()
    tr, ti, gamma = transition_parameters(params["radius_logit"], params["theta"])
    read = field_read(raw, tr, ti, gamma, field_chunk)
    out = F.linear(rms_norm(read, params["read_norm.weight"]),
                   params["out_proj.weight"], params["out_proj.bias"])
    gate = torch.sigmoid(F.linear(x, params["gate_proj.weight"], params["gate_proj.bias"]))
    return x + (out * gate).to(x.dtype)
