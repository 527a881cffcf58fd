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


def _softpatch_like(via_holder: bool):
    """A module laid out like the reference's softpatch mixers: ``FastBoundaryStateMixer`` finds
    the scan on a module it holds as ``v3_global``, ``BoundaryStateMixer`` as a global of its
    own file (official_source/field_hybrid_speed_optimization_v6.py:333-335 and
    field_hybrid_attentionfree_qualification_v3.py:460)."""
    import types
    calls = []

    def hierarchical_scan(a, b, block=32):
        calls.append((a.dtype, a.device.type))
        return b

    home = types.ModuleType("scan_home_for_test")
    home.hierarchical_scan = hierarchical_scan
    if via_holder:
        source = ("import torch\nv3_global = None\n"
                  "class FastBoundaryStateMixer(torch.nn.Module):\n"
                  "    def forward(self, a, b):\n"
                  "        return v3_global.hierarchical_scan(a, b, block=32)\n")
    else:
        source = ("import torch\n"
                  "class BoundaryStateMixer(torch.nn.Module):\n"
                  "    def forward(self, a, b):\n"
                  "        return hierarchical_scan(a, b, block=32)\n")
    user = types.ModuleType("scan_user_for_test")
    exec(source, user.__dict__)
    if via_holder:
        user.v3_global = home
        return user.FastBoundaryStateMixer(), home.__dict__, calls
    user.hierarchical_scan = hierarchical_scan
    return user.BoundaryStateMixer(), user.__dict__, calls


@pytest.mark.parametrize("via_holder", [True, False])
def test_install_scan_rebinds_where_the_softpatch_mixer_looks(via_holder):
    mixer, namespace, calls = _softpatch_like(via_holder)
    model = torch.nn.Sequential(mixer)
    original = namespace["hierarchical_scan"]
    assert fields_lm_b200.install_scan(model) == 1
    assert namespace["hierarchical_scan"] is not original
    assert namespace["hierarchical_scan"].__wrapped__ is original
    assert fields_lm_b200.install_scan(model) == 1          # idempotent: not wrapped twice
    assert namespace["hierarchical_scan"].__wrapped__ is original
    # CPU and complex calls still reach the reference's own function through the replacement
    a = torch.rand(1, 5, 3)
    mixer(a, a)
    mixer(a.to(torch.complex64), a.to(torch.complex64))
    assert calls == [(torch.float32, "cpu"), (torch.complex64, "cpu")]
    fields_lm_b200.uninstall(model)
    assert namespace["hierarchical_scan"] is original
    assert fields_lm_b200.install_scan(torch.nn.Linear(2, 2)) == 0
