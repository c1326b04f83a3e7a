"""The shared library loads on a CPU-only host and exports every symbol the header declares."""

import ctypes
import re
from pathlib import Path

from bongard_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def header_symbols():
    text = (ROOT / 'include' / 'bongard_b200.h').read_text()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(bg_\w+)\s*\(', text)))


def test_header_and_binding_agree():
    assert header_symbols() == _lib.declared_symbols()


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in header_symbols():
        assert hasattr(lib, name), name


def test_version_and_error_string_without_a_gpu():
    lib = _lib.load()
    assert lib.bg_version() >= 1
    assert isinstance(lib.bg_last_error_string(), bytes)
