"""The CUDA library builds, loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADERS = sorted((ROOT / "include").glob("*.h"))


def declared_functions():
    names = []
    for h in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names += re.findall(r"\b(fields_\w+)\s*\(", text)
    return sorted(set(names))


@pytest.fixture(scope="module")
def library():
    from fields_lm_b200 import build
    path = build.build_library()
    return ctypes.CDLL(str(path))


def test_header_declares_the_operator():
    names = declared_functions()
    for must in ("fields_read_forward", "fields_read_backward", "fields_read_workspace_bytes",
                 "fields_status_string"):
        assert must in names


def test_library_exports_every_declared_symbol(library):
    missing = [n for n in declared_functions() if not hasattr(library, n)]
    assert not missing, missing


def test_loader_binds_every_declared_symbol(library):
    from fields_lm_b200 import _lib
    assert sorted(_lib.SYMBOLS) == declared_functions()
    lib = _lib.load()
    assert lib.fields_read_version() >= 100
    assert lib.fields_status_string(0) == b"ok"
    # host-only queries work without a device
    assert lib.fields_read_workspace_bytes(8, 2048, 512, 0) > 0
    assert lib.fields_read_workspace_bytes(0, 2048, 512, 0) == 0


def test_emulation_and_library_agree_on_workspace(library):
    import emu
    from fields_lm_b200 import _lib
    lib = _lib.load()
    for dims in [(1, 1, 4), (8, 2048, 512), (1, 65536, 512), (3, 130, 20), (2, 33, 7)]:
        for which in (0, 1):
            assert lib.fields_read_workspace_bytes(*dims, which) == \
                emu.lib().fields_read_workspace_bytes(*dims, which)
