"""ctypes binding of libbongard_b200.so (the C ABI declared in include/bongard_b200.h).

There is no fallback: if the library is missing or a call fails, the error is raised.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / 'libbongard_b200.so'

P, I64, I32, F32, F64, INT = c_void_p, c_int64, c_int32, c_float, c_double, c_int

SIGNATURES = {
    'bg_version': ([], INT),
    'bg_last_error_string': ([], c_char_p),
    'bg_device_check': ([], INT),
    'bg_read_status': ([P], INT),
    'bg_selftest_bounded_wait': ([I64, P, P], INT),
    'bg_rmsnorm': ([P, I64, P, P, I64, I64, I64, F32, P], INT),
    'bg_add_rmsnorm': ([P, P, P, P, P, I64, I64, F32, P], INT),
    'bg_rmsnorm_f32': ([P, I64, P, P, I64, I64, I64, F32, P], INT),
    'bg_add_rmsnorm_f32': ([P, P, P, P, P, I64, I64, F32, P], INT),
    'bg_add_rmsnorm_f32y': ([P, P, P, P, P, I64, I64, F32, P], INT),
    'bg_gemm_bf16_f32out': ([P, I64, P, I64, P, I64, I64, I64, P], INT),
    'bg_embed_f32': ([P, P, P, P, I64, I64, F32, I64, I64, P], INT),
    'bg_qk_norm_rope': ([P, I64, INT, P, I64, INT, P, P, P, P, I64, INT, F32, INT, P], INT),
    'bg_qk_norm_rope_table': ([P, I64, INT, P, I64, INT, P, P, P, P, I64, INT, F32, P], INT),
    'bg_qk_norm_rope_cached': ([P, I64, INT, P, I64, INT, P, P, P, P, I64, I64, INT, F32, P], INT),
    'bg_embed': ([P, P, P, P, I64, I64, F32, I64, I64, P], INT),
    'bg_gemm_bf16': ([P, I64, P, I64, P, I64, I64, I64, I64, INT, P], INT),
    'bg_transpose_bf16': ([P, I64, P, I64, I64, I64, P], INT),
    'bg_geglu_backward': ([P, P, P, I64, I64, P], INT),
    'bg_geglu_forward': ([P, P, I64, I64, P], INT),
    'bg_rmsnorm_backward_workspace_bytes': ([I64, I64], I64),
    'bg_rmsnorm_backward': ([P, I64, P, P, I64, P, I64, P, P, I64, I64, I64, F32, P], INT),
    'bg_qk_norm_rope_backward_workspace_bytes': ([I64, INT], I64),
    'bg_qk_norm_rope_backward': ([P, I64, P, I64, P, I64, INT, P, I64, P, I64, P, I64, INT, P, P, P, P, P, P, P, P, P,
                                  I64, I64, INT, F32, INT, P], INT),
    'bg_set_programmatic_launch': ([INT], None),
    'bg_rope_table': ([P, I64, INT, P, P], INT),
    'bg_gemm_bf16_qkv_rope': ([P, I64, P, I64, P, I64, I64, I64, INT, INT, INT, P, P, P, P, I64, F32, P], INT),
    'bg_gemm_bf16_skinny_supported': ([I64, I64, I64, INT], INT),
    'bg_gemm_bf16_tn': ([P, I64, P, I64, P, I64, I64, I64, I64, INT, P, I64, P], INT),
    'bg_gemm_bf16_splitk_choice': ([I64, I64, I64], INT),
    'bg_gemm_bf16_splitk_workspace_bytes': ([I64, I64, INT], I64),
    'bg_gemm_bf16_splitk': ([P, I64, P, I64, P, I64, I64, I64, I64, INT, P, I64, P], INT),
    'bg_gemm_bf16_skinny': ([P, I64, P, I64, P, I64, I64, I64, I64, INT, P], INT),
    'bg_quantize_e4m3_rows': ([P, I64, P, I64, P, I64, I64, P], INT),
    'bg_quantize_e4m3_tiles': ([P, I64, P, I64, P, I64, I64, P], INT),
    'bg_gemm_fp8_block128': ([P, I64, P, P, I64, P, P, I64, I64, I64, I64, INT, P], INT),
    'bg_mxfp8_scale_bytes': ([I64, I64], I64),
    'bg_quantize_mxfp8': ([P, I64, P, I64, P, I64, I64, P], INT),
    'bg_gemm_mxfp8': ([P, I64, P, P, I64, P, P, I64, I64, I64, I64, INT, P], INT),
    'bg_rmsnorm_mxfp8': ([P, I64, P, P, P, I64, I64, F32, P], INT),
    'bg_add_rmsnorm_mxfp8': ([P, P, P, P, P, P, I64, I64, F32, P], INT),
    'bg_gemm_mxfp8_geglu_q': ([P, I64, P, P, I64, P, P, I64, P, I64, I64, I64, P], INT),
    'bg_linear_fp8_workspace_bytes': ([I64, I64], I64),
    'bg_linear_fp8': ([P, I64, P, I64, P, P, I64, I64, I64, I64, INT, P, I64, P], INT),
    'bg_linear_fp8_static_max_bytes': ([], I64),
    'bg_linear_fp8_static': ([P, I64, P, I64, P, P, I64, I64, I64, I64, INT, P], INT),
    'bg_attention_tile_rows': ([INT], INT),
    'bg_attention_item_index': ([INT, INT, INT], INT),
    'bg_attention_pair_tile_rows': ([INT], INT),
    'bg_varlen_attention': ([P, I64, I64, P, P, I64, I64, P, P, I64, I64, P, P, P, I32, P, P, I64, I64, I64, INT, INT, INT,
                             F32, P], INT),
    'bg_varlen_attention_pair': ([P, I64, I64, P, P, I64, I64, P, P, I64, I64, P, P, P, I32, P, P, I64, I64, I64, INT, INT, INT,
                             F32, P], INT),
    'bg_varlen_attention_backward': ([P, I64, I64, P, P, I64, I64, P, P, I64, I64, P, P, I64, I64, P, P, P, P, P, P, P,
                                      P, I32, P, I32, P, P, I64, I64, I64, INT, INT, INT, F32, P], INT),
    'bg_judgment_head': ([P, I64, P, P, P, P, P, P, I64, I64, INT, P], INT),
    'bg_candidate_softmax': ([P, P, P, I64, F64, P], INT),
}

_lib = None


class B200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def declared_symbols():
    return sorted(SIGNATURES)


def load():
    """Load the shared library once and declare every signature."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f'{LIB_PATH} is missing: build it with `python -m bongard_b200.build` '
                '(or __graft_entry__.build()); there is no fallback path')
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype
        _lib = lib
    return _lib


def check(code, what):
    if code != 0:
        message = load().bg_last_error_string().decode()
        if code in (-1, -2):
            raise ValueError(f'{what}: {message}')
        raise B200Error(f'{what} failed with status {code}: {message}')
