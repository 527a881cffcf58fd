"""Builds the reference's full 24-layer model from the staged copy. TEST INFRASTRUCTURE ONLY.

The promoted fields-lm model (18 native Field blocks, 2 Mamba-2 editors, 4 refresh-attention
blocks, PCAF cache, about 300 M parameters) is constructed by the reference's own public
function ``build_official_fields`` (``src/fields_official/fields_official.py:374-416``) from the
staged package under ``oracle/_ref``, untouched. Where ``mamba-ssm`` is not installed, the
labelled stand-in of :mod:`oracle.mamba_standin` takes the place of ``mamba_ssm.Mamba2`` before
the reference is imported; results obtained that way carry ``STANDIN_LABEL``.

Used by ``tests/test_gpu_full_model.py`` and by the ``full_model`` leg of ``bench.py`` to run one
training step with the reference's Triton Field kernels and one with this repository's CUDA
library installed, on the same model object (same weights), and compare loss and gradients.
"""
from __future__ import annotations

import contextlib
import sys
import tempfile
from pathlib import Path
from typing import Dict, Tuple

import torch

from . import mamba_standin, ref


def build(device, model_seed: int = 0):
    """Returns ``(model, standin_in_use)``: ``FieldsForCausalLM`` on ``device``, fp32 weights."""
    ref.verify()
    standin = mamba_standin.install()
    root = str(ref.REF_ROOT)
    if root not in sys.path:
        sys.path.insert(0, root)
    with contextlib.redirect_stdout(sys.stderr):  # the constructors print progress lines
        from fields_official import FieldsConfig, build_official_fields
        tmp = Path(tempfile.mkdtemp(prefix="fields_full_model_"))
        cfg = FieldsConfig(cache_dir=tmp / "hf", output_dir=tmp / "out", model_seed=int(model_seed))
        model = build_official_fields(cfg, device=device)
    return model, standin


def token_batch(batch: int, length: int, seed: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token ids uniform in [0, 16384) and next-token labels, as the reference's smoke test
    forms them (``scripts/smoke_test_h100.py:20-21``)."""
    gen = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 16_384, (batch, length), generator=gen, dtype=torch.long).to(device)
    return ids, torch.roll(ids, -1, 1)


def training_step(model, ids, labels) -> torch.Tensor:
    """One forward + backward under bf16 autocast through the public ``forward``; returns the loss."""
    model.zero_grad(set_to_none=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(ids, labels)
    out.loss.backward()
    return out.loss.detach().float()


def gradients(model) -> Dict[str, torch.Tensor]:
    return {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}


def compare_gradients(got: Dict[str, torch.Tensor], want: Dict[str, torch.Tensor]):
    """Worst per-tensor relative error ``max|a - b| / max(max|b|, 1e-6)`` (the reference's own
    gradient measure, ``field_only_v4_chunked_triton_wiki100.py:1448-1450``) and its tensor."""
    worst, worst_name = 0.0, ""
    for name, b in want.items():
        a = got[name]
        err = float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))
        if err > worst:
            worst, worst_name = err, name
    return worst, worst_name


def field_block_count(model) -> int:
    return sum(1 for m in model.modules() if type(m).__name__ == "IndependentVacancyField")
