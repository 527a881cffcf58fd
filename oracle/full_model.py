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


def norm_relative(got: Dict[str, torch.Tensor], want: Dict[str, torch.Tensor]):
    """Worst per-tensor ``||a - b||_2 / ||b||_2`` and its tensor: insensitive to single elements
    that a one-ulp bfloat16 flip moves."""
    worst, worst_name = 0.0, ""
    for name, b in want.items():
        d = float((got[name].double() - b.double()).norm() / b.double().norm().clamp_min(1e-12))
        if d > worst:
            worst, worst_name = d, name
    return worst, worst_name


def field_mixers(model):
    return [m for m in model.modules() if type(m).__name__ == "IndependentVacancyField"]


def set_triton_geometry(model, block_c: int, chunk_t: int) -> None:
    """Launch geometry of the reference's Triton kernels for every Field mixer. The reference
    treats its geometries as interchangeable ("exact", its own sweep:
    ``official_source/field_fusion_gap_closure_v33.py:4-6,38-41``; candidates
    ``official_source/field_fusion_gap_kernel_v32.py:836-847``). The channel block does not
    touch the arithmetic; a different chunk length composes the same recurrence in a
    different order, i.e. perturbs ``read`` at fp32 rounding level. Running the reference against itself that way measures how far such a perturbation
    travels through the 24 bf16 layers - the floor under any comparison of two exact kernels."""
    for m in field_mixers(model):
        m.triton_block_c, m.triton_chunk_t = int(block_c), int(chunk_t)


class ReadCapture:
    """Records ``read`` (the input of ``read_norm``) of every Field mixer during a forward."""

    def __init__(self, model):
        self.reads, self.handles = [], []
        for m in field_mixers(model):
            self.handles.append(m.read_norm.register_forward_pre_hook(
                lambda mod, args: self.reads.append(args[0].detach().float().clone())))

    def close(self):
        for h in self.handles:
            h.remove()


def reads_by_block(model, ids):
    """``read`` of each of the Field mixers, in block order, from one evaluation-mode forward
    under bf16 autocast (no checkpoint recomputation in evaluation mode)."""
    was_training = model.training
    model.eval()
    cap = ReadCapture(model)
    try:
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            model(ids)
    finally:
        cap.close()
        model.train(was_training)
    return cap.reads


def field_block_count(model) -> int:
    return sum(1 for m in model.modules() if type(m).__name__ == "IndependentVacancyField")
