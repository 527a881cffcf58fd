"""Re-points a built fields-lm model at the CUDA library, without touching its source.

The reference's Field mixer looks ``fused_field_read`` up as a global of its own
module at call time (``field_only_v4_chunked_triton_wiki100.py:1175-1183``).
Every model build executes that file into a fresh module object, so the patch is
applied per model: find the mixers, take the globals of their ``forward`` and
rebind the name. The reference files and their SHA-256 digests stay as they are,
and ``backend`` stays ``"triton"``.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .field_read import fused_field_read

_NAME = "fused_field_read"
_MIXER_CLASS = "IndependentVacancyField"
_saved: Dict[int, object] = {}


def _namespaces(model: torch.nn.Module) -> List[dict]:
    seen, out = set(), []
    for module in model.modules():
        if type(module).__name__ != _MIXER_CLASS:
            continue
        ns = type(module).forward.__globals__
        if id(ns) not in seen and _NAME in ns:
            seen.add(id(ns))
            out.append(ns)
    return out


def install(model: torch.nn.Module, fn=fused_field_read) -> int:
    """Rebinds ``fused_field_read`` for every Field mixer in ``model``.

    Returns the number of module namespaces patched (one per model build).
    Raises if the model holds no Field mixer with the Triton backend boundary.
    """
    spaces = _namespaces(model)
    if not spaces:
        raise ValueError("no IndependentVacancyField with a fused_field_read global in this model")
    for ns in spaces:
        _saved.setdefault(id(ns), ns[_NAME])
        ns[_NAME] = fn
    return len(spaces)


def uninstall(model: torch.nn.Module) -> int:
    """Restores the original operator in every namespace ``install`` changed."""
    n = 0
    for ns in _namespaces(model):
        if id(ns) in _saved:
            ns[_NAME] = _saved.pop(id(ns))
            n += 1
    return n
