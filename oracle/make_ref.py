"""Stages the reference's own Python package next to the oracle. TEST INFRASTRUCTURE ONLY.

``python oracle/make_ref.py --reference-root <checkout>`` copies ``src/fields_official``
of a fields-lm checkout, byte for byte, into ``oracle/_ref/fields_official`` (a git-ignored
folder: the files never enter this repository's history) and checks two things:

* the canonical Field module's SHA-256 equals the digest the checkout itself pins in
  ``SOURCE_IDENTITY.txt`` (``canonical_sha256=...``) and in
  ``src/fields_official/fields_official.py`` (``OFFICIAL_CANONICAL_SHA256``);
* every copied file is byte-identical to its source.

The staged copy lets the tests and the benchmark run the reference's own functions where
the checkout itself is absent: ``reference_field_read`` + autograd on the host cores (the
timed CPU baseline), the six Triton kernels behind ``fused_field_read`` on the same GPU
(the comparator), ``run_kernel_self_test`` and the reference's ``FieldBlock`` /
``IndependentVacancyField`` classes as the call site of ``fields_lm_b200.install``.
The shipped package never imports it.
"""
from __future__ import annotations

import argparse
import hashlib
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
PACKAGE_REL = Path("src") / "fields_official"
CANON_REL = PACKAGE_REL / "reference" / "field_only_v4_chunked_triton_wiki100.py"
IDENTITY = "SOURCE_IDENTITY.txt"


def sha256(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


def pinned_digest(root: Path) -> str:
    for line in (root / IDENTITY).read_text().splitlines():
        if line.startswith("canonical_sha256="):
            return line.split("=", 1)[1].strip()
    raise RuntimeError(f"{IDENTITY} holds no canonical_sha256 line")


def stage(root: Path, dest: Path = DEST) -> Path:
    """Copies the package and verifies it; returns the staged package directory."""
    root = root.resolve()
    src = root / PACKAGE_REL
    if not src.is_dir():
        raise FileNotFoundError(f"{src} is not a directory: not a fields-lm checkout")
    want = pinned_digest(root)
    got = sha256(root / CANON_REL)
    if got != want:
        raise RuntimeError(f"canonical module digest {got} differs from the pinned {want}")
    target = dest / "fields_official"
    if target.exists():
        shutil.rmtree(target)
    dest.mkdir(parents=True, exist_ok=True)
    shutil.copytree(src, target, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    shutil.copyfile(root / IDENTITY, dest / IDENTITY)
    n = 0
    for path in sorted(src.rglob("*")):
        if path.is_dir() or "__pycache__" in path.parts or path.suffix == ".pyc":
            continue
        copy = target / path.relative_to(src)
        if sha256(copy) != sha256(path):
            raise RuntimeError(f"{copy} differs from its source")
        n += 1
    (dest / "STAGED.txt").write_text(
        f"verbatim copy of {PACKAGE_REL} ({n} files)\ncanonical_sha256={got}\n")
    return target


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--reference-root", type=Path, required=True)
    args = ap.parse_args()
    target = stage(args.reference_root)
    print(f"staged {target} ({(DEST / 'STAGED.txt').read_text().splitlines()[0]})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
