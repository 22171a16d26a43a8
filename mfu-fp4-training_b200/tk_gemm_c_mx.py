"""Host-side mirror of the reference's ``_C_mx`` extension module (MXFP4 tcgen05 GEMMs):
fp4_runtime/ThunderKittens/kernels/gemm/mxfp4_gb200/mxfp4_gb200_gemm.cu:2704-3028.
``D = bf16((A . B^T) / 36)`` with E8M0 scales per 32 elements; ``D`` pre-allocated, returns None."""
from __future__ import annotations

import torch

from . import _lib
from .tk_gemm_c import _chk_operand, _chk_out, _shapes, _stream


def _gemm(A, A_sc, B, B_sc, D, residual=None):
    for t, n in ((A, "A"), (A_sc, "A_sc"), (B, "B"), (B_sc, "B_sc")):
        _chk_operand(t, n)
    M, N, K = _shapes(A, B)
    out_fp32 = 1 if D.dtype == torch.float32 else 0
    _chk_out(D, M, N, D.dtype if out_fp32 else torch.bfloat16)
    if residual is not None:
        _chk_out(residual, M, N)
    with torch.cuda.device(A.device):
        _lib.call("fp4b200_mxfp4_gemm", A.data_ptr(), A_sc.data_ptr(), B.data_ptr(), B_sc.data_ptr(), D.data_ptr(),
                  out_fp32, None if residual is None else residual.data_ptr(), M, N, K, _stream(A))


def mxfp4_gemm(A, A_sc, B, B_sc, D):
    _gemm(A, A_sc, B, B_sc, D)


def mxfp4_gemm_config(A, A_sc, B, B_sc, D, config_id):
    """``config_id`` is accepted and ignored: this library has one tile shape."""
    _gemm(A, A_sc, B, B_sc, D)


def mxfp4_gemm_residual(A, A_sc, B, B_sc, R, D):
    _gemm(A, A_sc, B, B_sc, D, residual=R)


def mxfp4_batched_gemm(A_list, A_sc_list, B_list, B_sc_list, D_out_list):
    for A, A_sc, B, B_sc, D in zip(A_list, A_sc_list, B_list, B_sc_list, D_out_list, strict=True):
        _gemm(A, A_sc, B, B_sc, D)


def mxfp4_batched_gemm_config(A_list, A_sc_list, B_list, B_sc_list, D_out_list, config_id):
    mxfp4_batched_gemm(A_list, A_sc_list, B_list, B_sc_list, D_out_list)
