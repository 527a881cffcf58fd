"""Generate the golden fixtures in this folder from the reference itself.

Run once, on a machine that has the reference checkout, with
``python tests/golden/make_golden.py --reference-root <checkout>``.
The script imports the reference's canonical Field module by file path (the
way the reference imports it itself), runs ``reference_field_read`` with
PyTorch autograd on CPU, and writes:

* ``op_small.npz``  — small and ragged operator cases, full tensors, forward
  and backward;
* ``config1.npz``   — one ``FieldBlock(1024, "reference", 32, 32, 64, 2528)``
  built under ``torch.manual_seed(0)``, input ``x ~ N(0,1)`` of shape
  ``[1, 256, 1024]``: the operator's inputs in full, its outputs every 4th
  step plus the last step, the mixer/block outputs every 4th step, and a hash
  of every weight so that a test can rebuild the same block from the seed;
* ``scan_small.npz`` — the reference's ``hierarchical_scan(a, b, 32)`` on real inputs with
  autograd: dense decays and one decay per token expanded over the channels (the softpatch
  mixer's call), ragged lengths around the block size of 32.

The fixtures travel with the repository; the reference does not.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
CANON_REL = "src/fields_official/reference/field_only_v4_chunked_triton_wiki100.py"

# (name, B, L, C, raw scale, parameter mode)
SMALL_CASES = [
    ("selftest_shape", 2, 37, 32, 1.0, "init"),
    ("single_step", 1, 1, 4, 1.0, "init"),
    ("ragged", 3, 130, 20, 1.5, "random"),
    ("one_chunk", 1, 64, 4, 1.0, "init"),
    ("chunk_plus_one", 2, 65, 12, 3.0, "random"),
    ("odd_channels", 2, 33, 7, 1.0, "random"),
    ("wide", 1, 48, 160, 0.6, "init"),
]


def load_canon(root: Path):
    path = root / CANON_REL
    spec = importlib.util.spec_from_file_location("fields_canon_for_golden", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod, hashlib.sha256(path.read_bytes()).hexdigest()


def init_parameters(C: int, mode: str, gen: torch.Generator):
    """radius_logit/theta as the mixer initialises them, or random ones."""
    if mode == "init":
        ring = torch.linspace(0.85, 0.999, C)
        radius_logit = torch.log(ring / (1.0 - ring))
        theta = torch.linspace(0.03, torch.pi * 0.97, C)
    else:
        radius_logit = torch.randn(C, generator=gen) * 2.5 + 1.0
        theta = (torch.rand(C, generator=gen) * 2.0 - 1.0) * torch.pi
    radius = torch.sigmoid(radius_logit).clamp(0.50, 0.99995).float()
    tr = radius * torch.cos(theta)
    ti = radius * torch.sin(theta)
    gamma = torch.sqrt((1.0 - radius.square()).clamp_min(1e-4))
    return tr, ti, gamma


def run_op(canon, raw, tr, ti, gamma, grad_read, field_chunk=32):
    raw = raw.clone().requires_grad_(True)
    tr = tr.clone().requires_grad_(True)
    ti = ti.clone().requires_grad_(True)
    gamma = gamma.clone().requires_grad_(True)
    read = canon.reference_field_read(raw, tr, ti, gamma, field_chunk)
    read.backward(grad_read)
    return read.detach(), raw.grad, tr.grad, ti.grad, gamma.grad


def make_small(canon) -> dict:
    out = {}
    gen = torch.Generator().manual_seed(20240607)
    for name, B, L, C, scale, mode in SMALL_CASES:
        tr, ti, gamma = init_parameters(C, mode, gen)
        raw = torch.randn(B, L, 3 * C, generator=gen) * scale
        grad_read = torch.randn(B, L, 4 * C, generator=gen)
        read, g_raw, g_tr, g_ti, g_gm = run_op(canon, raw, tr, ti, gamma, grad_read)
        for key, val in dict(raw=raw, tr=tr, ti=ti, gamma=gamma, grad_read=grad_read,
                             read=read, grad_raw=g_raw, grad_tr=g_tr, grad_ti=g_ti,
                             grad_gamma=g_gm).items():
            out[f"{name}/{key}"] = val.numpy().astype(np.float32)
    out["cases"] = np.array([c[0] for c in SMALL_CASES])
    return out


# (name, B, L, C, decay per token broadcast over the channels?, range of a)
SCAN_CASES = [
    ("softpatch_shape", 2, 70, 64, True, (0.01, 0.99)),
    ("single_step", 1, 1, 3, False, (0.0, 1.0)),
    ("ragged_dense", 3, 45, 5, False, (0.0, 1.0)),
    ("one_block", 1, 32, 8, True, (0.01, 0.99)),
    ("block_plus_one", 2, 33, 40, True, (0.01, 0.99)),
    ("signed_decay", 2, 100, 33, False, (-1.0, 1.0)),
]


def make_scan(canon) -> dict:
    out = {}
    gen = torch.Generator().manual_seed(20240609)
    for name, B, L, C, per_token, (lo, hi) in SCAN_CASES:
        shape = (B, L) if per_token else (B, L, C)
        a0 = (lo + (hi - lo) * torch.rand(shape, generator=gen)).requires_grad_(True)
        a = a0[..., None].expand(B, L, C) if per_token else a0
        b = torch.randn(B, L, C, generator=gen).requires_grad_(True)
        g = torch.randn(B, L, C, generator=gen)
        states = canon.hierarchical_scan(a, b, 32)
        states.backward(g)
        for key, val in (("a", a0), ("b", b), ("grad_states", g), ("states", states),
                         ("grad_a", a0.grad), ("grad_b", b.grad)):
            out[f"{name}/{key}"] = val.detach().numpy().copy()
    out["cases"] = np.array([c[0] for c in SCAN_CASES])
    return out


def weight_digest(module: torch.nn.Module) -> str:
    h = hashlib.sha256()
    for name, p in sorted(module.state_dict().items()):
        h.update(name.encode())
        h.update(p.detach().contiguous().numpy().tobytes())
    return h.hexdigest()


def make_config1(canon) -> dict:
    torch.manual_seed(0)
    block = canon.FieldBlock(1024, "reference", 32, 32, 64, 2528)
    block.eval()
    gen = torch.Generator().manual_seed(1)
    # rounded to fp16 so that the stored half-precision copy is exact
    x = torch.randn(1, 256, 1024, generator=gen).half().float()
    mixer = block.mixer
    with torch.no_grad():
        raw = mixer.write_proj(x).contiguous().float()
        radius = torch.sigmoid(mixer.radius_logit).clamp(0.50, 0.99995).float()
        theta = mixer.theta.float()
        tr = radius * torch.cos(theta)
        ti = radius * torch.sin(theta)
        gamma = torch.sqrt((1.0 - radius.square()).clamp_min(1e-4))
        mixed = mixer(x)
        y = block(x)
    grad_read = torch.randn(1, 256, 2048, generator=gen).half().float()
    read, g_raw, g_tr, g_ti, g_gm = run_op(canon, raw, tr, ti, gamma, grad_read)
    keep = sorted(set(range(0, 256, 4)) | {255})
    return {
        "x": x.numpy().astype(np.float16), "raw": raw.numpy(), "tr": tr.numpy(), "ti": ti.numpy(),
        "gamma": gamma.numpy(), "grad_read": grad_read.numpy().astype(np.float16),
        "steps": np.array(keep, dtype=np.int64),
        "read_steps": read[:, keep].numpy(), "grad_raw_steps": g_raw[:, keep].numpy(),
        "grad_tr": g_tr.numpy(), "grad_ti": g_ti.numpy(), "grad_gamma": g_gm.numpy(),
        "mixer_out_steps": mixed[:, keep].numpy(), "block_out_steps": y[:, keep].numpy(),
        "weight_sha256": np.array(weight_digest(block)),
        "ff_hidden": np.array(2528),
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", required=True, type=Path)
    ap.add_argument("--only-scan", action="store_true", help="write scan_small.npz only")
    args = ap.parse_args()
    torch.set_num_threads(1)  # fixed reduction order inside the reference's GEMMs
    canon, sha = load_canon(args.reference_root)
    scan = make_scan(canon)
    scan["canon_sha256"] = np.array(sha)
    np.savez_compressed(HERE / "scan_small.npz", **scan)
    print("scan_small.npz", (HERE / "scan_small.npz").stat().st_size, "bytes")
    if args.only_scan:
        return
    small = make_small(canon)
    small["canon_sha256"] = np.array(sha)
    np.savez_compressed(HERE / "op_small.npz", **small)
    cfg1 = make_config1(canon)
    cfg1["canon_sha256"] = np.array(sha)
    np.savez_compressed(HERE / "config1.npz", **cfg1)
    for f in ("op_small.npz", "config1.npz"):
        print(f, (HERE / f).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
