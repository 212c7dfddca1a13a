"""ctypes binding of libspgt_b200.so (the C ABI declared in include/spgt_b200.h).

There is no fallback: if the library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, 'libspgt_b200.so')

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f'{LIB_PATH} is missing: build it with `python -m spgt_b200.build` (needs nvcc). '
        'spgt_b200 has no CPU or PyTorch fallback.')

lib = C.CDLL(LIB_PATH)

_f = C.c_void_p      # device pointer
_i = C.c_int
_fl = C.c_float
_sz = C.c_size_t
_st = C.c_void_p     # cudaStream_t

SIGNATURES = {
    'spgt_error_string': (C.c_char_p, [_i]),
    'spgt_last_cuda_error': (_i, []),
    'spgt_abi_version': (_i, []),
    'spgt_set_tuning': (_i, [C.c_char_p, _i]),
    'spgt_projpos_fwd': (_i, [_f, _f, _f, _f, _f, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_projpos_lnorm_fwd': (_i, [_f, _f, _f, _f, _f, _fl, _f, _f, _f, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_projpos_qkv_fwd': (_i, [_f] * 11 + [_fl] + [_f] * 4 + [_i] * 6 + [_st]),
    'spgt_galerkin_attn_fwd': (_i, [_f, _f, _f, _f, _f, _i, _i, _i, _i, _i, _st]),
    'spgt_galerkin_attn_bwd_workspace_bytes': (_sz, [_i, _i, _i, _i]),
    'spgt_galerkin_attn_bwd': (_i, [_f, _f, _f, _f, _f, _f, _f, _i, _i, _i, _i, _f, _sz, _st]),
    'spgt_projpos_bwd_workspace_bytes': (_sz, [_i, _i, _i]),
    'spgt_projpos_bwd_elementwise': (_i, [_f, _f, _f, _fl, _f, _f, _f, _f, _i, _i, _i, _i, _i, _f, _sz, _st]),
    'spgt_skinny_gemm_workspace_bytes': (_sz, [_i, _i, _i, _i]),
    'spgt_batched_skinny_gemm': (_i, [_f, _f, _f, _fl, _i, _i, _i, _i, _f, _sz, _st]),
    'spgt_skinny_gemm_noalloc_max_bytes': (_sz, []),
    'spgt_batched_skinny_gemm_noalloc': (_i, [_f, _f, _f, _fl, _i, _i, _i, _i, _st]),
    'spgt_ffn_tc_fwd': (_i, [_f, _i, _f, _f, _f, _f, _f, _i, _f, _i, _i, _i, _i, _i, _st]),
    'spgt_relative_l2_fwd': (_i, [_f, _f, _f, _i, C.c_int64, _fl, _st]),
    'spgt_darcy_fv_workspace_bytes': (C.c_size_t, [_i, _i]),
    'spgt_darcy_fv_solve': (_i, [_f, _f, _f, _i, _i, _i, C.c_double, _i, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, _st]),
    'spgt_batched_transpose': (_i, [_f, _f, _i, _i, _i, _st]),
    'spgt_transpose_gather_dual': (_i, [_f, _f, _f] + [_i] * 9 + [_st]),
    'spgt_transpose_scatter_dual': (_i, [_f, _f, _f] + [_i] * 9 + [_st]),
    'spgt_linear_fwd': (_i, [_f, _i, _f, _i, _f, _f, _i, _f, _i, _i, _i, _i, _i, _st]),
    'spgt_conv3x3_fwd': (_i, [_f, _i, _i, _i, _f, _i, _f, _f, _i, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_bilinear_fwd': (_i, [_f, _f, _i, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_bilinear_concat3_fwd': (_i, [_f, _f, _f] + [_i] * 6 + [_f] + [_i] * 6 + [_st]),
    'spgt_conv0_down_fwd': (_i, [_f, _f, _f, _f, _i, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_upsample_grid_fwd': (_i, [_f, _f, _f, _f, _f, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_decoder_head_fwd': (_i, [_f, _f, _f, _f, _fl, _fl, _fl, _f, _f, _i, _f, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_tc_weight_bytes': (_sz, [_i, _i]),
    'spgt_tc_weight_prepare': (_i, [_f, _i, _i, _i, _f, _sz, _st]),
    'spgt_tc_status': (_i, []),
    'spgt_tc_status_reset': (_i, []),
    'spgt_tc_selftest_wait_expiry': (_i, [_i, _i, _f, _st]),
    'spgt_linear_tc_fwd': (_i, [_f, _i, _f, _f, _f, _i, _f, _i, _i, _i, _i, _i, _st]),
    'spgt_conv3x3_tc_fwd': (_i, [_f, _i, _i, _i, _f, _f, _f, _i, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_projpos_qkv_tc_fwd': (_i, [_f] * 9 + [_fl] + [_f] * 4 + [_i] * 6 + [_st]),
    'spgt_decoder_head_tc_fwd': (_i, [_f, _f, _f, _f, _fl, _fl, _fl, _f, _f, _i, _f, _i, _i, _i, _i, _i, _i, _st]),
    'spgt_spectral_tables_bytes': (_sz, [_i, _i]),
    'spgt_spectral_tables_init': (_i, [_f, _sz, _i, _i, _st]),
    'spgt_spectral_workspace_bytes': (_sz, [_i, _i, _i, _i]),
    'spgt_spectral_chunk_samples': (_i, [_i]),
    'spgt_spectral_launches': (_i, [_i, _i, _i]),
    'spgt_spectral_conv2d_fwd': (_i, [_f, _f, _f, _f, _f, _f, _f, _sz, _f, _i, _i, _i, _i, _i, _st]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)       # AttributeError here = the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


class SpgtError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib.spgt_error_string(code).decode()
        cuda = lib.spgt_last_cuda_error() if code == -5 else 0
        super().__init__(f'{where}: {msg} (code {code}' + (f', cudaError {cuda})' if cuda else ')'))


def check(code: int, where: str) -> None:
    if code != 0:
        raise SpgtError(code, where)
