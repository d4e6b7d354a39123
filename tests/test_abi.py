"""The C-ABI library loads and exports every symbol ``include/nvq.h`` declares, and
the ctypes signature table lists exactly those symbols (no compute calls here)."""
import ctypes
import os
import re

from novann_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "nvq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(nvq_[a-z0-9_]+)\s*\(", text))


def test_header_matches_signature_table():
    assert _declared() == set(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    assert os.path.exists(_lib.LIB_PATH), "build with python -m novann_b200.build"
    L = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in _declared() if not hasattr(L, n)]
    assert not missing, missing


def test_version_and_error_string():
    L = _lib.lib()
    assert b"sm_100a" in L.nvq_version()
    assert isinstance(L.nvq_last_error(), bytes)


def test_argument_validation_needs_no_gpu():
    # cols not a multiple of 32 is rejected before any CUDA call
    L = _lib.lib()
    st = L.nvq_quantize_fp4_b32(None, None, None, 4, 40, 0, None)
    assert st == _lib.ERR_INVALID
    assert b"multiple of 32" in L.nvq_last_error()
    st = L.nvq_quantize_fp8(None, None, 16, _lib.E4M3, ctypes.c_float(0.0), 0, None)
    assert st == _lib.ERR_INVALID
