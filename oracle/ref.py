"""Loads the staged copy of the reference (``oracle/_ref``). TEST INFRASTRUCTURE ONLY.

``oracle/make_ref.py`` puts a verbatim, digest-checked copy of the reference's
``src/fields_official`` package under ``oracle/_ref``. This module executes the
canonical Field module of that copy the way the reference does itself: by file path,
into a FRESH module object on every call
(``official_source/field_scale_50m_v15.py:36-44``), so each caller owns the module
globals it may re-point (``fused_field_read``).

Used by the tests, the smoke check and the benchmark only.
"""
from __future__ import annotations

import hashlib
import importlib.util
import itertools
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_ROOT = HERE / "_ref"
PACKAGE = REF_ROOT / "fields_official"
CANON = PACKAGE / "reference" / "field_only_v4_chunked_triton_wiki100.py"
_counter = itertools.count()


def available() -> bool:
    return CANON.is_file() and (REF_ROOT / "SOURCE_IDENTITY.txt").is_file()


def why_unavailable() -> str:
    return (f"{CANON.relative_to(HERE.parent)} is missing: run `python oracle/make_ref.py "
            "--reference-root <fields-lm checkout>` where the checkout exists")


def pinned_digest() -> str:
    for line in (REF_ROOT / "SOURCE_IDENTITY.txt").read_text().splitlines():
        if line.startswith("canonical_sha256="):
            return line.split("=", 1)[1].strip()
    raise RuntimeError("SOURCE_IDENTITY.txt holds no canonical_sha256 line")


def verify() -> str:
    """Checks the staged canonical module against the digest the reference pins; returns it."""
    if not available():
        raise FileNotFoundError(why_unavailable())
    got = hashlib.sha256(CANON.read_bytes()).hexdigest()
    want = pinned_digest()
    if got != want:
        raise RuntimeError(f"staged canonical module digest {got} differs from the pinned {want}")
    return got


def load_canon(name: str | None = None):
    """Executes the staged canonical Field module into a new module object and returns it."""
    verify()
    name = name or f"fields_canon_staged_{next(_counter)}"
    spec = importlib.util.spec_from_file_location(name, CANON)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod  # dataclasses in the module look their module up by name
    spec.loader.exec_module(mod)
    return mod


def selftest_args(canon):
    """The argparse namespace ``run_kernel_self_test`` expects, with the reference's defaults
    (tolerances ``field_only_v4_chunked_triton_wiki100.py:2280-2283``)."""
    argv, sys.argv = sys.argv, ["field_only_v4_chunked_triton_wiki100.py"]
    try:
        return canon.parse_args()
    finally:
        sys.argv = argv
