"""A labelled STAND-IN for ``mamba_ssm.Mamba2``. TEST INFRASTRUCTURE ONLY.

The reference's full 24-layer model holds two Mamba-2 editor blocks
(``official_source/field_fusion_wiki100_mamba2_v25.py:73-91``) built from the
``mamba-ssm`` package (version 2.3.2.post1) and ``causal-conv1d``, neither of which is
installed here. They are outside the path this repository replaces; they only surround
it when the whole model runs. ``install()`` registers stand-in modules under both names
BEFORE the reference is imported, so that the reference's constructors, its shape solver
and its topology audit run unchanged:

* same constructor keywords as the reference passes
  (``d_model, d_state, d_conv, expand, headdim, ngroups, chunk_size, use_mem_eff_path``);
* the same parameter tensors, names and shapes as the published Mamba-2 layer
  (``in_proj``, depth-wise ``conv1d``, ``dt_bias``, ``A_log``, ``D``, ``norm.weight``,
  ``out_proj``), so the parameter count, and with it the solved model shape, is the one
  the real package gives;
* a simple causal forward that is NOT Mamba-2: a gated causal depth-wise convolution
  with a per-head scalar gain. No line of mamba-ssm is reproduced.

Every result obtained with it is labelled "Mamba-2 editors replaced by stand-in"; both
sides of such a comparison (the reference's Triton Field path and this repository's CUDA
path) use the same stand-in, so it cancels out of the comparison.
"""
from __future__ import annotations

import sys
import types

import torch
import torch.nn as nn
import torch.nn.functional as F

STANDIN_LABEL = "Mamba-2 editors replaced by stand-in: mamba-ssm unavailable"
REPORTED_VERSION = "2.3.2.post1"  # the version string the reference's arena checks for


class _GatedNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x, z):
        x = x * F.silu(z)
        return F.rms_norm(x.float(), (x.shape[-1],), self.weight.float(), self.eps).to(x.dtype)


class Mamba2(nn.Module):
    """Stand-in with the parameter shapes of a Mamba-2 layer and a simple causal forward."""

    def __init__(self, d_model, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1,
                 chunk_size=256, use_mem_eff_path=True, **unused):
        super().__init__()
        self.d_model, self.d_state, self.d_conv = int(d_model), int(d_state), int(d_conv)
        self.d_inner = int(expand) * self.d_model
        self.headdim, self.ngroups = int(headdim), int(ngroups)
        if self.d_inner % self.headdim:
            raise ValueError("expand * d_model must be a multiple of headdim")
        self.nheads = self.d_inner // self.headdim
        conv_dim = self.d_inner + 2 * self.ngroups * self.d_state
        self.in_proj = nn.Linear(self.d_model, 2 * self.d_inner + 2 * self.ngroups * self.d_state
                                 + self.nheads, bias=False)
        self.conv1d = nn.Conv1d(conv_dim, conv_dim, self.d_conv, groups=conv_dim,
                                padding=self.d_conv - 1, bias=True)
        self.dt_bias = nn.Parameter(torch.zeros(self.nheads))
        self.A_log = nn.Parameter(torch.zeros(self.nheads))
        self.D = nn.Parameter(torch.ones(self.nheads))
        self.norm = _GatedNorm(self.d_inner)
        self.out_proj = nn.Linear(self.d_inner, self.d_model, bias=False)

    def forward(self, u):
        B, L, _ = u.shape
        z, xbc, dt = torch.split(
            self.in_proj(u),
            [self.d_inner, self.d_inner + 2 * self.ngroups * self.d_state, self.nheads], dim=-1)
        xbc = F.silu(self.conv1d(xbc.transpose(1, 2))[..., :L].transpose(1, 2))  # causal
        x = xbc[..., :self.d_inner].reshape(B, L, self.nheads, self.headdim)
        gain = torch.sigmoid(dt.float() + self.dt_bias.float()) * torch.exp(-torch.exp(
            self.A_log.float())) + self.D.float()
        y = (x * gain.unsqueeze(-1).to(x.dtype)).reshape(B, L, self.d_inner)
        return self.out_proj(self.norm(y, z))


def install() -> bool:
    """Registers the stand-in as ``mamba_ssm`` / ``causal_conv1d`` unless the real packages
    import. Returns True if the stand-in is in use. Call before importing the reference."""
    try:
        import causal_conv1d  # noqa: F401
        import mamba_ssm  # noqa: F401
        return bool(getattr(mamba_ssm, "FIELDS_STANDIN", False))
    except Exception:
        pass
    m = types.ModuleType("mamba_ssm")
    m.Mamba2 = Mamba2
    m.__version__ = REPORTED_VERSION
    m.FIELDS_STANDIN = True
    c = types.ModuleType("causal_conv1d")
    c.__version__ = "stand-in"
    c.FIELDS_STANDIN = True
    sys.modules["mamba_ssm"] = m
    sys.modules["causal_conv1d"] = c
    return True
