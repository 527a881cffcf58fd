"""Mirror of the reference's Field mixer and Field block, for tests that run where the staged
reference is absent. TEST INFRASTRUCTURE.

Same parameters, names, initialisation order and arithmetic as ``IndependentVacancyField`` and
``FieldBlock`` (``field_only_v4_chunked_triton_wiki100.py:300-325, 1131-1221``), so a
``state_dict`` moves between the two unchanged and a block built under the same seed holds the
same weights. The forward looks ``fused_field_read`` up as a global of this module, like the
reference's, so ``fields_lm_b200.install`` can be exercised on it. With the staged reference at
hand the tests in ``test_gpu_reference.py`` use the reference's own classes instead.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from fields_lm_b200 import mixer as fm
from fields_lm_b200.field_read import fused_field_read  # rebound by install()


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        return (xf * inv * self.weight.float()).to(x.dtype)


class PackedSwiGLU(nn.Module):
    def __init__(self, dim: int, hidden: Optional[int] = None):
        super().__init__()
        self.hidden = int(hidden) if hidden is not None else ((int(8 * dim / 3) + 63) // 64) * 64
        self.w12 = nn.Linear(dim, 2 * self.hidden, bias=False)
        self.w3 = nn.Linear(self.hidden, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gate, value = self.w12(x).chunk(2, dim=-1)
        return self.w3(F.silu(gate) * value)


class IndependentVacancyField(nn.Module):
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
        # test switches (not constructor arguments: the signature mirrors the reference's)
        self.bf16_io = False     # keep the write projection's bf16 output under autocast
        self.fused_norm = False  # with bf16_io: run fused_mixer_forward where it applies

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.bf16_io and self.fused_norm:
            y = fm.fused_mixer_forward(self, x)
            if y is not None:
                return y
        if self.bf16_io:
            y = fm.bf16_mixer_forward(self, x)
            if y is not None:
                return y
        raw = self.write_proj(x).contiguous().float()
        tr, ti, gamma = fm.transition_parameters(self.radius_logit, self.theta)
        read = fused_field_read(raw, tr, ti, gamma, self.triton_block_c, self.triton_chunk_t)
        out = self.out_proj(self.read_norm(read))
        return x + (out * torch.sigmoid(self.gate_proj(x))).to(x.dtype)


class FieldBlock(nn.Module):
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

    def prefill(self, x: torch.Tensor):
        return fm.block_prefill(self, x)

    def step(self, x: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        return fm.block_step(self, x, state)
