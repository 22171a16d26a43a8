"""ctypes wrapper of the C restatement (oracle/fp4_oracle.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "libfp4oracle.so")
_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            subprocess.run(["make", "-s", "-C", HERE], check=True)
        _lib = ctypes.CDLL(LIB)
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def num_threads() -> int:
    return load().oracle_num_threads()


def fused_norm_quantize(x_bits, gamma_bits, eps, inv_rms=None, encode_centric=True, want_col=True):
    """x_bits uint16 [M,K] (bf16 bit patterns).  Returns dict like the numpy oracle."""
    lib = load()
    M, K = x_bits.shape
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    gamma_bits = np.ascontiguousarray(gamma_bits, dtype=np.uint16)
    compute = inv_rms is None
    inv = np.empty(M, dtype=np.float32) if compute else np.ascontiguousarray(inv_rms, dtype=np.float32).copy()
    normed = np.empty((M, K), dtype=np.uint16)
    row_fp4 = np.empty((M, K // 2), dtype=np.uint8)
    row_sc = np.empty((M // 128, K // 64, 512), dtype=np.uint8)
    col_fp4 = np.empty((K, M // 2), dtype=np.uint8) if want_col else None
    col_sc = np.empty((K // 128, M // 64, 512), dtype=np.uint8) if want_col else None
    amax_sg = np.zeros(2, dtype=np.float32)
    rc = lib.oracle_fused_norm_quantize(_ptr(x_bits), _ptr(gamma_bits), ctypes.c_float(eps), ctypes.c_int64(M),
                                        ctypes.c_int64(K), _ptr(inv), int(compute), int(encode_centric),
                                        _ptr(normed), _ptr(row_fp4), _ptr(row_sc), _ptr(col_fp4), _ptr(col_sc),
                                        _ptr(amax_sg))
    assert rc == 0
    return dict(row_fp4=row_fp4, row_sc=row_sc, col_fp4=col_fp4, col_sc=col_sc, inv_rms=inv,
                amax=amax_sg[0], sg=amax_sg[1])


def quantize_for_gemm(x_bits, encode_centric=True, want_col=True):
    lib = load()
    M, K = x_bits.shape
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    row_fp4 = np.empty((M, K // 2), dtype=np.uint8)
    row_sc = np.empty((M // 128, K // 64, 512), dtype=np.uint8)
    col_fp4 = np.empty((K, M // 2), dtype=np.uint8) if want_col else None
    col_sc = np.empty((K // 128, M // 64, 512), dtype=np.uint8) if want_col else None
    amax_sg = np.zeros(2, dtype=np.float32)
    rc = lib.oracle_quantize_for_gemm(_ptr(x_bits), ctypes.c_int64(M), ctypes.c_int64(K), int(encode_centric),
                                      _ptr(row_fp4), _ptr(row_sc), _ptr(col_fp4), _ptr(col_sc), _ptr(amax_sg))
    assert rc == 0
    return dict(row_fp4=row_fp4, row_sc=row_sc, col_fp4=col_fp4, col_sc=col_sc, amax=amax_sg[0], sg=amax_sg[1])
