"""ctypes binding of libfp4b200.so.  There is no fallback: if the library is missing or a
call fails, a RuntimeError is raised."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfp4b200.so")
if os.environ.get("FP4B200_LIB"):
    LIB_PATH = os.environ["FP4B200_LIB"]   # another build of the same library (A/B timing)

_c_void_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_f32 = ctypes.c_float

# name -> argtypes; every function returns int (0 = ok) unless listed in _RESTYPES
SIGNATURES = {
    "fp4b200_last_error": [],
    "fp4b200_abi_version": [],
    "fp4b200_device_status": [],
    "fp4b200_nvfp4_amax": [_c_void_p, _i64, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize": [_c_void_p, _i64, _i64, _c_void_p, _c_void_p, _int, _c_void_p, _c_void_p,
                               _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize_for_gemm": [_c_void_p, _i64, _i64, _int, _int, _c_void_p, _c_void_p, _c_void_p,
                                        _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize_opt": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _c_void_p, _c_void_p, _int, _int, _int,
                                   _int, _int, ctypes.c_uint64, ctypes.c_uint64, _int, ctypes.c_uint64,
                                   ctypes.c_uint64, ctypes.c_uint64, _c_void_p, _int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                   _c_void_p, _c_void_p],
    "fp4b200_sr_prepare_state": [_c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, _c_void_p],
    "fp4b200_sr_reserve_from_state": [_c_void_p, _c_void_p, ctypes.c_uint64, _c_void_p],
    "fp4b200_sr_set_invocation_offset": [ctypes.c_uint64, _c_void_p],
    "fp4b200_sr_get_invocation_offset": [_c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize_opt_into": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _c_void_p, _c_void_p, _int, _int, _int,
                                        _int, _int, ctypes.c_uint64, ctypes.c_uint64, _int, ctypes.c_uint64,
                                        ctypes.c_uint64, ctypes.c_uint64, _c_void_p, _int, _c_void_p, _i64, _c_void_p, _c_void_p,
                                        _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_rht16_amax": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _int, _int, ctypes.c_uint64, ctypes.c_uint64, _c_void_p,
                                 _c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize_weight_2d": [_c_void_p, _i64, _i64, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                         _c_void_p],
    "fp4b200_nvfp4_quantize_weight_2d_with_amax": [_c_void_p, _i64, _i64, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                                   _c_void_p],
    "fp4b200_nvfp4_rmsnorm_stats": [_c_void_p, _c_void_p, _f32, _i64, _i64, _c_void_p, _int, _c_void_p,
                                    _c_void_p],
    "fp4b200_nvfp4_fused_norm_quantize": [_c_void_p, _c_void_p, _f32, _i64, _i64, _c_void_p, _int, _int,
                                          _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize_normed": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _i64, _i64, _int, _c_void_p,
                                      _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_fused_norm_quantize_noalloc": [_c_void_p, _c_void_p, _f32, _i64, _i64, _c_void_p, _c_void_p,
                                                  _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_quantize": [_c_void_p, _i64, _i64, _int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_quantize_normed": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _int, _c_void_p, _c_void_p,
                                      _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_rmsnorm_inv_rms": [_c_void_p, _c_void_p, _f32, _i64, _i64, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_rmsnorm_inv_rms_opt": [_c_void_p, _c_void_p, _f32, _i64, _i64, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_silu_mul_quantize": [_c_void_p, _c_void_p, _i64, _i64, _int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                        _c_void_p],
    "fp4b200_mxfp4_quantize_nhsd_wo": [_c_void_p, _i64, _i64, _i64, _i64, _int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                       _c_void_p],
    "fp4b200_mxfp4_quantize_split": [ctypes.POINTER(_c_void_p), ctypes.POINTER(_i64), _int, _i64, _int, _c_void_p, _c_void_p,
                                     _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_quantize_split3_inverse_rope": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _i64, _i64, _c_void_p, _i64,
                                                   _int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_silu_mul_quantize_strided": [_c_void_p, _i64, _i64, _i64, _i64, _int, _c_void_p, _c_void_p, _c_void_p,
                                                _c_void_p, _c_void_p],
    "fp4b200_mxfp4_silu_deriv_quantize_split2": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _int, _c_void_p, _c_void_p,
                                                 _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_silu_deriv_quantize_split2_combined": [_c_void_p, _i64, _c_void_p, _i64, _i64, _i64, _i64, _int,
                                                          _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_silu_deriv_quantize_split2_splitcols": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _int, _c_void_p,
                                                           _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_selftest_silu_division": [_c_void_p, _c_void_p],
    "fp4b200_silu_mul_bf16": [_c_void_p, _c_void_p, _i64, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_silu_quantize": [_c_void_p, _c_void_p, _i64, _i64, _c_void_p, _int, _c_void_p, _c_void_p,
                                    _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_silu_deriv_bf16": [_c_void_p, _c_void_p, _c_void_p, _i64, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                _c_void_p],
    "fp4b200_set_gemm_pdl": [_int],
    "fp4b200_selftest_bounded_wait": [_i64, _c_void_p],
    "fp4b200_set_pdl_early_reads": [_int],
    "fp4b200_nvfp4_gemm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _int,
                           _c_void_p, _i64, _i64, _i64, _c_void_p],
    "fp4b200_nvfp4_gemm_accum": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                 _int, _i64, _i64, _i64, _c_void_p],
    "fp4b200_nvfp4_batched_accum_gemm": [_int, ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p),
                                         ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p),
                                         ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64), _c_void_p, _i64, _i64,
                                         _int, _c_void_p],
    "fp4b200_nvfp4_grouped_gemm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _int,
                                   ctypes.POINTER(_c_void_p), ctypes.POINTER(_i64), _i64, _i64, _i64, _c_void_p],
    "fp4b200_mxfp4_gemm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _int, _c_void_p, _i64, _i64,
                           _i64, _c_void_p],
    "fp4b200_mxfp4_gemm_rope": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _i64, _i64, _i64, _i64, _i64,
                                _c_void_p],
    "fp4b200_mxfp4_gemm_ksplit": [_c_void_p, _i64, _int, ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                                  ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p), ctypes.POINTER(_c_void_p),
                                  _c_void_p, _int, _i64, _i64, _c_void_p],
    "fp4b200_mxfp4_gemm_ksplit_strided": [_c_void_p, _i64, _int, ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                                          ctypes.POINTER(_c_void_p), ctypes.POINTER(_i64), ctypes.POINTER(_c_void_p),
                                          ctypes.POINTER(_c_void_p), _c_void_p, _int, _i64, _i64, _c_void_p],
    "fp4b200_mxfp4_quantize_weight_2d": [_c_void_p, _i64, _i64, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_quantize_row_sr": [_c_void_p, _i64, _i64, _int, _int, _int, _int, _int, ctypes.c_uint64, ctypes.c_uint64, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_mxfp4_quantize_row_and_col_sr": [_c_void_p, _i64, _i64, _int, _int, _int, _int, _int, _int, _int, ctypes.c_uint64,
                                              ctypes.c_uint64, _c_void_p,
                                              _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_row_rms_reduce": [_c_void_p, _i64, _i64, _i64, _f32, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize_for_gemm_into": [_c_void_p, _i64, _i64, _int, _int, _c_void_p, _i64, _c_void_p, _c_void_p, _c_void_p,
                                             _c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize_split3_into": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _i64, _i64, _c_void_p, _c_void_p,
                                           _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_quantize_nhsd_wo": [_c_void_p, _i64, _i64, _i64, _i64, _int, _int, _c_void_p, _c_void_p, _c_void_p,
                                       _c_void_p, _c_void_p, _c_void_p],
    "fp4b200_nvfp4_grouped_gemm_rope": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _int, _c_void_p,
                                        _c_void_p, _c_void_p, _i64, _i64, _i64, _int, _i64, _i64, _i64, _i64, _c_void_p],
    "fp4b200_rope_packed_qk": [_c_void_p, _c_void_p, _c_void_p, _i64, _i64, _c_void_p, _c_void_p, _i64, _i64, _i64, _int,
                               _c_void_p],
    "fp4b200_sum3_rmsnorm_bwd": [_c_void_p] * 10 + [_int, _i64, _i64, _c_void_p],
    "fp4b200_rmsnorm_bwd_residual": [_c_void_p] * 8 + [_i64, _i64, _c_void_p],
    "fp4b200_fp32_to_fp4x2": [_c_void_p, _i64, _c_void_p, _c_void_p],
    "fp4b200_fp4x2_to_fp32": [_c_void_p, _i64, _c_void_p, _c_void_p],
    "fp4b200_tk_nvfp4_quantize": [_c_void_p, _i64, _i64, _c_void_p, _c_void_p, _c_void_p, _int, _c_void_p],
}
_RESTYPES = {"fp4b200_last_error": ctypes.c_char_p}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library (once) and declares every prototype of include/fp4b200.h."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(HERE, 'build.py')}` "
            "(there is no CPU or PyTorch fallback for the FP4 hot path)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, _int)
    _lib = lib
    return lib


def call(name: str, *args) -> None:
    """Calls an int-returning entry point and raises RuntimeError with the library's message."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.fp4b200_last_error()
        raise RuntimeError(f"{name} failed: {msg.decode() if msg else rc}")


def device_status() -> int:
    return load().fp4b200_device_status()
