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


def test_argument_checks_need_no_device(library):
    """Bad arguments are refused with a status code before anything is launched."""
    from fields_lm_b200 import _lib
    lib = _lib.load()
    ARG, UNSUPPORTED = 1, 5
    assert lib.fields_read_state_rows(2048) == 256 and lib.fields_read_state_rows(7) == 0
    assert lib.fields_mixer_epilogue_bias_rows(16384) == 1024
    assert lib.fields_mixer_epilogue_forward(None, None, None, None, None, None, None, 1e-6, 2048,
                                             4, 8, None) == ARG
    assert lib.fields_mixer_epilogue_backward(None, None, None, None, None, None, None, None, None,
                                              None, None, 1e-6, 2048, 4, 8, None) == ARG
    assert lib.fields_read_norm_grad_combine(None, None, None, None, 4, 8, None) == ARG
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    # a feature count that is not a multiple of four
    assert lib.fields_read_norm_grad_combine(p, p, p, p, 4, 6, None) == UNSUPPORTED
    assert lib.fields_read_backward_from_states(None, None, None, None, None, None, None, None,
                                                None, None, None, None, None, None, 0, 1, 8, 4,
                                                None) == ARG
    assert lib.fields_read_forward_bf16_stats(None, None, None, None, None, None, None, None, None,
                                              0, 1, 8, 4, None) == ARG
    assert lib.fields_read_span_summary_backward(None, None, None, None, None, None, 0, 1, 8, 4,
                                                 None) == ARG
