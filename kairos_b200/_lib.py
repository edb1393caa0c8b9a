"""ctypes binding of libkairos_b200.so (the C ABI declared in include/kairos_b200.h).

There is no fallback: if the shared library is missing, importing this module raises,
and every compute entry point raises on a non-zero status.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libkairos_b200.so')

c_void_p, c_int, c_size_t, c_char_p = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_char_p
c_u64_p = ctypes.POINTER(ctypes.c_uint64)

# name -> (restype, argtypes); mirrors include/kairos_b200.h one to one
SIGNATURES = {
    'kairos_abi_version': (c_int, []),
    'kairos_status_str': (c_char_p, [c_int]),
    'kairos_last_error': (c_char_p, []),
    'kairos_device_status': (c_int, [c_int]),
    'kairos_selftest_bounded_wait': (c_int, [c_void_p]),
    'kairos_set_arithmetic': (c_int, [c_int]),
    'kairos_get_arithmetic': (c_int, []),
    'kairos_act_quant_i8': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    'kairos_w4_to_w8': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    'kairos_w4_to_f16': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    'kairos_awq_to_qserve': (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    'kairos_w4a16_gemv': (c_int, [c_void_p] * 6 + [c_int] * 3 + [c_void_p]),
    'kairos_w4a16_decode': (c_int, [c_void_p] * 6 + [c_int] * 3 + [c_void_p]),
    'kairos_w4a16_decode_silu': (c_int, [c_void_p] * 6 + [c_int] * 3 + [c_void_p]),
    'kairos_silu_mul_blocked': (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    'kairos_silu_mul_quant_blocked': (c_int, [c_void_p] * 4 + [c_int, c_int, c_void_p]),
    'kairos_w4a16_small_batch': (c_int, [c_void_p] * 6 + [c_int] * 3 + [c_void_p]),
    'kairos_gemm_workspace_bytes': (c_size_t, [c_int, c_int, c_int]),
    'kairos_gemm_plan_query': (c_int, [c_int, c_int, c_int, c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                                       ctypes.POINTER(c_int)]),
    'kairos_w4a16_gemm': (c_int, [c_void_p] * 6 + [c_int] * 3 + [c_void_p, c_size_t, c_void_p]),
    'kairos_w4a16_gemm_noalloc': (c_int, [c_void_p] * 6 + [c_int] * 3 + [c_void_p]),
    'kairos_w8a16_gemm': (c_int, [c_void_p] * 5 + [c_int] * 3 + [c_void_p, c_size_t, c_void_p]),
    'kairos_w8a8_gemm': (c_int, [c_void_p] * 7 + [c_int] * 3 + [c_void_p, c_size_t, c_void_p]),
    'kairos_f16_gemm': (c_int, [c_void_p] * 4 + [c_int] * 3 + [c_void_p, c_size_t, c_void_p]),
    'kairos_rms_norm': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_float, c_void_p]),
    'kairos_silu_mul': (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    'kairos_rms_norm_quant': (c_int, [c_void_p] * 6 + [c_int, c_int, ctypes.c_float, c_void_p]),
    'kairos_add_rms_norm': (c_int, [c_void_p] * 4 + [c_int, c_int, ctypes.c_float, c_void_p]),
    'kairos_silu_mul_quant': (c_int, [c_void_p] * 4 + [c_int, c_int, c_void_p]),
    'kairos_rope_kv': (c_int, [c_void_p] * 4 + [c_int] + [c_void_p] * 3 + [c_int] * 6 + [c_void_p]),
    'kairos_peer_allreduce_signal_bytes': (c_int, []),
    'kairos_peer_allreduce_f16': (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, ctypes.c_longlong, c_void_p]),
    'kairos_add_rms_norm_peer': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                         ctypes.c_float, c_void_p]),
    'kairos_rms_norm_quant_peer': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_int, ctypes.c_float, c_void_p]),
    'kairos_lut_create': (c_void_p, []),
    'kairos_lut_destroy': (None, [c_void_p]),
    'kairos_lut_record': (c_int, [c_void_p, c_int, c_int]),
    'kairos_lut_get': (c_int, [c_void_p, c_int]),
    'kairos_lut_shrink_to_fit': (None, [c_void_p]),
    'kairos_lut_size': (c_int, [c_void_p]),
    'kairos_ctx_create': (c_void_p, [c_size_t]),
    'kairos_ctx_destroy': (None, [c_void_p]),
    'kairos_ctx_reserve': (c_int, [c_void_p, c_int, c_int, c_int]),
    'kairos_ctx_stats': (c_int, [c_void_p, c_u64_p, c_u64_p, c_u64_p, c_u64_p]),
    'kairos_ctx_clear_cache': (None, [c_void_p]),
    'kairos_layer_create': (c_void_p, [c_void_p, c_int, c_int] + [c_void_p] * 7),
    'kairos_layer_destroy': (None, [c_void_p]),
    'kairos_switched_linear': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    'kairos_switched_linear_q8': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    'kairos_layer_prefetch': (c_int, [c_void_p, c_int, c_void_p]),
    'kairos_switched_linear_host': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f'{LIB_PATH} is missing: build the CUDA extension first (python -m kairos_b200.build). '
        'This package has no CPU or eager fallback.')

lib = ctypes.CDLL(LIB_PATH)
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)       # AttributeError here = header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args

SIZE_MAX = ctypes.c_size_t(-1).value


class KairosError(RuntimeError):
    pass


def check(status, what=''):
    """Raise KairosError for a negative status code of the C ABI."""
    if status is not None and status < 0:
        msg = lib.kairos_status_str(status).decode()
        detail = lib.kairos_last_error().decode()
        raise KairosError(f'{what}: {msg} (status {status})' + (f' [{detail}]' if detail else ''))
    return status
