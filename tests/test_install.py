"""install() rebinds the operator at the reference's own call site (CPU)."""
import importlib.util
import os
import sys
from pathlib import Path

import pytest
import torch

import fields_lm_b200
import mirror

CANON_REL = "src/fields_official/reference/field_only_v4_chunked_triton_wiki100.py"


def test_install_on_mirror_block_routes_calls():
    block = mirror.FieldBlock(16, "triton", 8, 8, 16, 32)
    calls = []

    def probe(raw, tr, ti, gamma, block_c, chunk_t):
        calls.append((tuple(raw.shape), raw.dtype, block_c, chunk_t, tr.requires_grad))
        return raw.new_zeros(raw.shape[0], raw.shape[1], 4 * tr.numel())

    assert fields_lm_b200.install(block, probe) == 1
    try:
        block(torch.randn(2, 5, 16))
    finally:
        assert fields_lm_b200.uninstall(block) == 1
    assert calls == [((2, 5, 24), torch.float32, 8, 16, True)]
    assert mirror.fused_field_read is fields_lm_b200.fused_field_read


def test_operator_rejects_cpu_and_wrong_dtype_like_the_reference():
    raw = torch.zeros(1, 2, 12)
    p = torch.zeros(4)
    with pytest.raises(RuntimeError, match="requires CUDA"):
        fields_lm_b200.fused_field_read(raw, p, p, p, 32, 64)


def _load_canon():
    """The reference's canonical module: the staged copy, else FIELDS_LM_REFERENCE, else a
    checkout named ``reference`` beside this repository. None if there is none."""
    from oracle import ref
    if ref.available():
        return ref.load_canon()
    sibling = Path(__file__).resolve().parent.parent.parent / "reference"
    for cand in (os.environ.get("FIELDS_LM_REFERENCE", ""), str(sibling)):
        if cand and (Path(cand) / CANON_REL).exists():
            spec = importlib.util.spec_from_file_location("canon_for_install_test",
                                                          Path(cand) / CANON_REL)
            canon = importlib.util.module_from_spec(spec)
            sys.modules[spec.name] = canon
            spec.loader.exec_module(canon)
            return canon
    return None


def test_install_on_the_reference_modules():
    canon = _load_canon()
    if canon is None:
        pytest.skip("neither the staged reference nor a checkout is present")
    block = canon.FieldBlock(16, "triton", 8, 8, 16, 32)
    original = canon.fused_field_read
    seen = []

    def probe(raw, tr, ti, gamma, block_c, chunk_t):
        seen.append((block_c, chunk_t))
        return canon.reference_field_read(raw, tr, ti, gamma, 8)

    assert fields_lm_b200.install(block, probe) == 1
    y = block(torch.randn(1, 6, 16))
    assert seen == [(8, 16)] and y.shape == (1, 6, 16)
    # the real operator is what install() binds by default, and it refuses CPU tensors
    fields_lm_b200.install(block)
    with pytest.raises(RuntimeError, match="requires CUDA"):
        block(torch.randn(1, 6, 16))
    assert fields_lm_b200.uninstall(block) == 1
    assert canon.fused_field_read is original


def test_install_fused_mixer_wraps_and_restores_the_class_forward():
    """fused_mixer=True replaces the mixer class's forward by a wrapper that falls back to the
    original one where the fused path does not apply (here: CPU), and uninstall restores it."""
    block = mirror.FieldBlock(16, "triton", 8, 8, 16, 32)
    cls = type(block.mixer)
    original = cls.forward
    calls = []

    def probe(raw, tr, ti, gamma, block_c, chunk_t):
        calls.append(tuple(raw.shape))
        return raw.new_zeros(raw.shape[0], raw.shape[1], 4 * tr.numel())

    x = torch.randn(2, 5, 16)
    try:
        assert fields_lm_b200.install(block, probe, fused_mixer=True) == 1
        assert cls.forward is not original
        y = block(x)                      # CPU: the wrapper hands over to the original forward
        assert calls == [(2, 5, 24)] and y.shape == x.shape
        assert fields_lm_b200.install(block, probe, fused_mixer=True) == 1   # idempotent
    finally:
        assert fields_lm_b200.uninstall(block) == 1
    assert cls.forward is original
    assert mirror.fused_field_read is fields_lm_b200.fused_field_read
