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


def header_prototypes():
    """name -> list of parameter type strings, read from the header's declarations."""
    text = (ROOT / 'include' / 'bongard_b200.h').read_text()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    out = {}
    for ret, name, params in re.findall(r'([\w\s\*]+?)\b(bg_\w+)\s*\(([^)]*)\)\s*;', text):
        params = params.strip()
        out[name] = [] if params in ('', 'void') else [' '.join(p.split()) for p in params.split(',')]
        out[name + ':ret'] = ' '.join(ret.split())
    return out


def kind(ctype):
    if ctype is None:
        return 'void'
    if ctype in (ctypes.c_void_p, ctypes.c_char_p):
        return 'pointer'
    if ctype in (ctypes.c_float, ctypes.c_double):
        return 'float' if ctype is ctypes.c_float else 'double'
    return {ctypes.c_int: 'int', ctypes.c_int32: 'int', ctypes.c_int64: 'int64'}[ctype]


def c_kind(decl):
    """Kind of one C parameter or return type, e.g. 'const void* q' -> pointer, 'int64_t ldq' -> int64."""
    if '*' in decl:
        return 'pointer'
    words = decl.replace('const', '').split()
    base = words[0] if words else 'void'
    return {'int': 'int', 'int32_t': 'int', 'int64_t': 'int64', 'float': 'float', 'double': 'double',
            'void': 'void'}[base]


def test_every_binding_has_the_headers_argument_list():
    """A ctypes signature with one argument too few, or an int where the header says int64_t, corrupts a
    call silently: the binding table is compared with the prototypes, argument by argument."""
    protos = header_prototypes()
    for name, (args, ret) in _lib.SIGNATURES.items():
        assert name in protos, name
        want = [c_kind(p) for p in protos[name]]
        got = [kind(a) for a in args]
        assert got == want, (name, got, want)
        assert kind(ret) == c_kind(protos[name + ':ret']), (name, ret, protos[name + ':ret'])
