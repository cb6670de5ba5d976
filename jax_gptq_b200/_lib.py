"""ctypes binding of libjgq.so (the C ABI declared in include/jgq.h).

There is no fallback: if the shared library is missing or does not export a
declared symbol, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, 'libjgq.so')

F32, F16, BF16, U8, I32 = 0, 1, 2, 3, 4
STATUS_NOT_PD, STATUS_NAN, STATUS_TIMEOUT = 1, 2, 4
W4_TRANSPOSE_B, W4_WEIGHTS_SETTLED = 1, 2

_i64, _int, _vp, _sz = C.c_int64, C.c_int, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); mirrors include/jgq.h one to one
SIGNATURES = {
    'jgq_version': (_int, []),
    'jgq_last_error': (C.c_char_p, []),
    'jgq_launch_count': (C.c_uint64, []),
    'jgq_pack_int4': (_int, [_vp, _int, _vp, _i64, _i64, _i64, _vp]),
    'jgq_unpack_int4': (_int, [_vp, _vp, _i64, _i64, _i64, _vp]),
    'jgq_pack_matrix': (_int, [_vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    'jgq_unpack_matrix': (_int, [_vp, _vp, _vp, _vp, _int, _i64, _i64, _i64, _vp]),
    'jgq_pack_int3': (_int, [_vp, _int, _vp, _i64, _i64, _i64, _vp]),
    'jgq_unpack_int3': (_int, [_vp, _vp, _i64, _i64, _i64, _vp]),
    'jgq_repack_int3_to_int4': (_int, [_vp, _vp, _i64, _i64, _i64, _vp]),
    'jgq_unpack_matrix3': (_int, [_vp, _vp, _vp, _vp, _int, _i64, _i64, _i64, _vp]),
    'jgq_col_params': (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    'jgq_hessian_workspace_bytes': (_sz, [_i64, _i64, _int]),
    'jgq_hessian_accum': (_int, [_vp, _int, _i64, _i64, _vp, _vp, _sz, _vp, _vp]),
    'jgq_hessian_finalize': (_int, [_vp, _i64, C.c_double, _vp]),
    'jgq_hessian_lower_elems': (_sz, [_i64]),
    'jgq_hessian_pack_lower': (_int, [_vp, _i64, _vp, _vp]),
    'jgq_hessian_unpack_lower': (_int, [_vp, _i64, _vp, _vp]),
    'jgq_permute_sym': (_int, [_vp, _i64, _vp, _vp, _vp]),
    'jgq_gather_rows': (_int, [_vp, _i64, _i64, _vp, _vp, _vp]),
    'jgq_damp_invert_workspace_bytes': (_sz, [_i64]),
    'jgq_damp_invert': (_int, [_vp, _i64, _vp, _i64, C.c_float, _vp, _vp, _sz, _vp, _vp]),
    'jgq_hessian_accum_f64': (_int, [_vp, _int, _i64, _i64, _vp, _vp]),
    'jgq_hessian_finalize_f64': (_int, [_vp, _i64, C.c_double, _vp]),
    'jgq_damp_invert_f64_workspace_bytes': (_sz, [_i64]),
    'jgq_damp_invert_f64': (_int, [_vp, _i64, _vp, _i64, C.c_double, _vp, _vp, _sz, _vp, _vp]),
    'jgq_gptq_quantize_workspace_bytes': (_sz, [_i64, _i64, _int]),
    'jgq_gptq_quantize': (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _vp, _int, _vp, _vp, _sz, _vp]),
    'jgq_w4_matmul_workspace_bytes': (_sz, [_i64, _i64, _i64, _int]),
    'jgq_w4_matmul': (_int, [_vp, _int, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    'jgq_w4_matmul_noalloc_max_bytes': (_sz, []),
    'jgq_w4_matmul_noalloc': (_int, [_vp, _int, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]),
}


class JgqError(RuntimeError):
    """A C-ABI call returned a negative status (nothing was launched)."""

    def __init__(self, code, message):
        super().__init__(f'jgq error {code}: {message}')
        self.code = code


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f'{LIB_PATH} not found: build it with `python -m jax_gptq_b200.build` '
            '(nvcc, sm_100a). There is no CPU or PyTorch fallback for this library.')
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)     # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc):
    if rc != 0:
        raise JgqError(rc, lib.jgq_last_error().decode('utf-8', 'replace'))
