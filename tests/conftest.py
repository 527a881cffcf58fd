"""Shared pytest configuration: the ``gpu`` marker, repo root on sys.path, fixtures."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"

# Tolerances of the parity contract. Relative error is max|x - ref| / max(max|ref|, 1e-6),
# the form the reference uses for its own gradient check
# (field_only_v4_chunked_triton_wiki100.py:1448-1450).
FP32_TOL = 1e-5
BF16_TOL = 2e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def rel_err(x, ref) -> float:
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if ref.size == 0:
        return 0.0
    return float(np.max(np.abs(x - ref)) / max(float(np.max(np.abs(ref))), 1e-6))


@pytest.fixture(scope="session")
def golden_small():
    return np.load(GOLDEN / "op_small.npz")


@pytest.fixture(scope="session")
def golden_config1():
    return np.load(GOLDEN / "config1.npz")


@pytest.fixture
def variants_library(monkeypatch):
    """Routes the package through the test build of the CUDA library, which also holds the
    measured kernel alternatives and picks them per call from FIELDS_READ_ALGO /
    FIELDS_FWD_VARIANT / FIELDS_BWD_VARIANT / FIELDS_READ_PREFETCH / FIELDS_READ_PDL. The product
    library reads none of these per call."""
    from fields_lm_b200 import _lib, build
    path = build.VARIANTS_LIB if build.VARIANTS_LIB.exists() else build.build_variants()
    monkeypatch.setattr(_lib, "_lib", _lib.open_library(path))
    return path
