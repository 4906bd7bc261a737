"""The C-ABI library loads, exports every symbol the header declares, and rejects bad arguments before touching the GPU."""
import ctypes
import re
from pathlib import Path

import pytest

from qwen_tailor_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "gdn_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:gdn|gqa)_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    syms = declared_symbols()
    for s in ("gdn_recurrent", "gdn_deltanet", "gdn_deltanet_b", "gdn_deltanet_bm", "gqa_decode_paged", "gdn_state_copy", "gdn_gates"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for s in declared_symbols():
        assert hasattr(lib, s), f"libgdn_b200.so does not export {s}"
        assert s in _lib.SIGNATURES, f"{s} has no ctypes prototype"
    assert lib.gdn_version() >= 100


def test_bad_shapes_are_rejected_without_a_device():
    lib = _lib.load()
    one = ctypes.c_void_p(16)
    rc = lib.gdn_recurrent(one, one, one, one, one, None, one, one, 1, 1, 16, 16, 64, 64, None)      # Dk = 64
    assert rc == -1 and b"Dk=128" in lib.gdn_last_error_string()
    with pytest.raises(ValueError):
        _lib.check(rc, "gdn_recurrent")
    assert lib.gdn_state_copy(one, one, 3, 4, 0, 0, 1, 0, 0, None) == -2                               # element size 3
    assert lib.gdn_state_copy(None, one, 4, 4, 0, 0, 1, 0, 0, None) == -8
    assert lib.gqa_decode_paged(one, one, one, one, one, one, one, one, one, 0, 1, 5, 16, 1, 1, 16, None) == -1   # M = 5
    assert lib.gdn_deltanet_b(one, 100, one, one, one, one, one, one, one, 4, one, 1, None) == -1      # row stride < 8224
    assert lib.gqa_decode_workspace_bytes(16, 8192) > 0
