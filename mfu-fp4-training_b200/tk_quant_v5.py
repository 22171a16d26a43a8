"""Host-side mirror of the reference's ``_tk_quant_v5`` extension module (NVFP4 producers).

Same function names, argument order, defaults, return tuples and error behaviour
(``RuntimeError`` on a rejected argument) as the pybind module defined at
fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:10815-11153.  Outputs are allocated with
torch on the input's device, kernels are enqueued on torch's current stream of that device
through the C ABI in ``include/fp4b200.h``.  There is no fallback path.
"""
from __future__ import annotations

import torch

from . import _lib

_FP4 = torch.float4_e2m1fn_x2
_E4M3 = torch.float8_e4m3fn


def _check_bf16_2d(t: torch.Tensor, name: str, mult: int = 128):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.bfloat16:
        raise RuntimeError(f"{name} must be bfloat16")
    if t.dim() != 2 or not t.is_contiguous():
        raise RuntimeError(f"{name} must be a contiguous 2-D tensor")
    M, K = t.shape
    if M % mult or K % mult:
        raise RuntimeError(f"{name}: M and K must be multiples of {mult} (got {M}x{K})")
    return M, K


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def _alloc_operands(M, K, device, want_col):
    u8 = dict(dtype=torch.uint8, device=device)
    row_fp4 = torch.empty((M, K // 2), **u8)
    row_sc = torch.empty((M // 128, K // 64, 512), **u8)
    if want_col:
        col_fp4 = torch.empty((K, M // 2), **u8)
        col_sc = torch.empty((K // 128, M // 64, 512), **u8)
    else:
        col_fp4 = torch.empty((0,), **u8)
        col_sc = torch.empty((0,), **u8)
    return row_fp4, row_sc, col_fp4, col_sc


def tk_quantize_for_gemm(input, return_transpose, encode_centric=True):
    """tk_quantize.cu:2208-2412 — returns (row_fp4, row_sc, col_fp4, col_sc, sg, sg, amax_buf, sync_buf)."""
    M, K = _check_bf16_2d(input, "input")
    with torch.cuda.device(input.device):
        row_fp4, row_sc, col_fp4, col_sc = _alloc_operands(M, K, input.device, return_transpose)
        amax_sg = torch.empty(2, dtype=torch.float32, device=input.device)
        sync_buf = torch.zeros(4, dtype=torch.int32, device=input.device)
        _lib.call("fp4b200_nvfp4_quantize_for_gemm", input.data_ptr(), M, K, int(bool(return_transpose)),
                  int(bool(encode_centric)), row_fp4.data_ptr(), row_sc.data_ptr(),
                  _p(col_fp4) if return_transpose else None, _p(col_sc) if return_transpose else None,
                  amax_sg.data_ptr(), _stream(input))
    sg = amax_sg.narrow(0, 1, 1)
    return (row_fp4.view(_FP4), row_sc.view(_E4M3), col_fp4.view(_FP4) if return_transpose else col_fp4,
            col_sc.view(_E4M3) if return_transpose else col_sc, sg, sg, amax_sg, sync_buf)


def _fused_norm_impl(input, gamma, eps, with_silu, return_transpose, inv_rms):
    M, K = _check_bf16_2d(input, "input")
    if with_silu:
        raise RuntimeError("tk_fused_norm_quantize: with_silu=True is not on the FFN hot path and is not built")
    if not isinstance(gamma, torch.Tensor) or gamma.dtype != torch.bfloat16 or gamma.numel() != K \
            or not gamma.is_contiguous() or gamma.device != input.device:
        raise RuntimeError("gamma must be contiguous CUDA bfloat16 [K] on the input device")
    compute = inv_rms is None
    if compute:
        inv_rms = torch.empty(M, dtype=torch.float32, device=input.device)
    else:
        if (not inv_rms.is_cuda or inv_rms.dtype != torch.float32 or inv_rms.dim() != 1
                or inv_rms.size(0) != M or not inv_rms.is_contiguous()):
            raise RuntimeError("inv_rms must be contiguous CUDA float32 [M]")
        if inv_rms.device != input.device:
            raise RuntimeError("inv_rms must be on the input device")
    with torch.cuda.device(input.device):
        row_fp4, row_sc, col_fp4, col_sc = _alloc_operands(M, K, input.device, return_transpose)
        amax_sg = torch.empty(2, dtype=torch.float32, device=input.device)
        _lib.call("fp4b200_nvfp4_fused_norm_quantize", input.data_ptr(), gamma.data_ptr(), float(eps), M, K,
                  inv_rms.data_ptr(), int(compute), 1, row_fp4.data_ptr(), row_sc.data_ptr(),
                  _p(col_fp4) if return_transpose else None, _p(col_sc) if return_transpose else None,
                  amax_sg.data_ptr(), _stream(input))
    return (row_fp4.view(_FP4), row_sc.view(_E4M3), col_fp4.view(_FP4) if return_transpose else col_fp4,
            col_sc.view(_E4M3) if return_transpose else col_sc, amax_sg.narrow(0, 1, 1), inv_rms,
            amax_sg.narrow(0, 0, 1), amax_sg, amax_sg)


def tk_fused_norm_quantize(input, gamma, epsilon, with_silu, return_transpose):
    """tk_quantize.cu:8003-8243 — returns (row_fp4, row_sc, col_fp4, col_sc, sg, inv_rms, amax, keep, keep);
    encode-centric, as the reference's default branch."""
    return _fused_norm_impl(input, gamma, epsilon, with_silu, return_transpose, None)


def tk_fused_norm_quantize_from_inv_rms(input, gamma, inv_rms, with_silu, return_transpose):
    """tk_quantize.cu:8250-8259 — as above with caller-provided inverse RMS."""
    return _fused_norm_impl(input, gamma, 0.0, with_silu, return_transpose, inv_rms)
