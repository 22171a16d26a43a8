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


def tk_quantize_weight_2d(input):
    """tk_quantize.cu:2445-2555 — 16x16-tile weight quantisation, returns
    (row_fp4, row_sc, col_fp4, col_sc, sg, sg)."""
    N, K = _check_bf16_2d(input, "input")
    with torch.cuda.device(input.device):
        row_fp4, row_sc, col_fp4, col_sc = _alloc_operands(N, K, input.device, True)
        amax_sg = torch.empty(2, dtype=torch.float32, device=input.device)
        _lib.call("fp4b200_nvfp4_quantize_weight_2d", input.data_ptr(), N, K, row_fp4.data_ptr(), row_sc.data_ptr(),
                  col_fp4.data_ptr(), col_sc.data_ptr(), amax_sg.data_ptr(), _stream(input))
    sg = amax_sg.narrow(0, 1, 1)
    return row_fp4.view(_FP4), row_sc.view(_E4M3), col_fp4.view(_FP4), col_sc.view(_E4M3), sg, sg


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


def _same_shape_bf16(ref, *others):
    for t in others:
        if (not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous()
                or t.shape != ref.shape or t.device != ref.device):
            raise RuntimeError("all inputs must be contiguous CUDA bfloat16 tensors of the same shape and device")


def tk_silu_mul_split_bf16(h1_raw, h3):
    """tk_quantize.cu (helper): ``bf16(silu(h1_raw) * h3)``."""
    _check_bf16_2d(h1_raw, "h1_raw", 8)
    _same_shape_bf16(h1_raw, h3)
    with torch.cuda.device(h1_raw.device):
        out = torch.empty_like(h1_raw)
        amax_sg = torch.empty(2, dtype=torch.float32, device=h1_raw.device)
        _lib.call("fp4b200_silu_mul_bf16", h1_raw.data_ptr(), h3.data_ptr(), h1_raw.numel(), out.data_ptr(),
                  amax_sg.data_ptr(), _stream(h1_raw))
    return out


def tk_silu_quantize_split_for_gemm(h1_raw, h3):
    """tk_quantize.cu:8985-9123 — returns (row_fp4, row_sc, col_fp4, col_sc, sg, sg, amax, sync, h_bf16);
    encode-centric like the reference's phase-2 template."""
    M, H = _check_bf16_2d(h1_raw, "h1_raw")
    _same_shape_bf16(h1_raw, h3)
    with torch.cuda.device(h1_raw.device):
        row_fp4, row_sc, col_fp4, col_sc = _alloc_operands(M, H, h1_raw.device, True)
        h = torch.empty_like(h1_raw)
        amax_sg = torch.empty(2, dtype=torch.float32, device=h1_raw.device)
        sync_buf = torch.zeros(4, dtype=torch.int32, device=h1_raw.device)
        _lib.call("fp4b200_nvfp4_silu_quantize", h1_raw.data_ptr(), h3.data_ptr(), M, H, h.data_ptr(), 1,
                  row_fp4.data_ptr(), row_sc.data_ptr(), col_fp4.data_ptr(), col_sc.data_ptr(), amax_sg.data_ptr(),
                  _stream(h1_raw))
    sg = amax_sg.narrow(0, 1, 1)
    return (row_fp4.view(_FP4), row_sc.view(_E4M3), col_fp4.view(_FP4), col_sc.view(_E4M3), sg, sg,
            amax_sg.narrow(0, 0, 1), sync_buf, h)


def _silu_deriv(dh, h3, h1_raw):
    M, H = _check_bf16_2d(dh, "dh")
    _same_shape_bf16(dh, h3, h1_raw)
    dev = dh.device
    dh1 = torch.empty_like(dh)
    dh3 = torch.empty_like(dh)
    a1 = torch.empty(2, dtype=torch.float32, device=dev)
    a3 = torch.empty(2, dtype=torch.float32, device=dev)
    _lib.call("fp4b200_silu_deriv_bf16", dh.data_ptr(), h3.data_ptr(), h1_raw.data_ptr(), dh.numel(),
              dh1.data_ptr(), dh3.data_ptr(), a1.data_ptr(), a3.data_ptr(), _stream(dh))
    return M, H, dh1, dh3, a1, a3


def tk_silu_deriv_split_bf16(dh, h3, h1_raw):
    """``(dh1, dh3)`` as bf16 (helper of the reference's backward producer)."""
    with torch.cuda.device(dh.device):
        _, _, dh1, dh3, _, _ = _silu_deriv(dh, h3, h1_raw)
    return dh1, dh3


def _quantize_with_amax(x, M, K, amax_sg, encode_centric, want_col=True):
    row_fp4, row_sc, col_fp4, col_sc = _alloc_operands(M, K, x.device, want_col)
    _lib.call("fp4b200_nvfp4_quantize", x.data_ptr(), M, K, amax_sg.data_ptr(), None, int(bool(encode_centric)),
              row_fp4.data_ptr(), row_sc.data_ptr(), _p(col_fp4) if want_col else None,
              _p(col_sc) if want_col else None, None, _stream(x))
    if want_col:
        return row_fp4.view(_FP4), row_sc.view(_E4M3), col_fp4.view(_FP4), col_sc.view(_E4M3)
    return row_fp4.view(_FP4), row_sc.view(_E4M3), col_fp4, col_sc


def tk_silu_deriv_quantize_split_for_gemm(dh, h3, h1_raw):
    """tk_quantize.cu:9418-9640 — 16-tuple: dh1 (row_fp4,row_sc,col_fp4,col_sc,sg,zero), dh3 likewise,
    amax buffer, sync buffer, dh1 bf16, dh3 bf16.  Encode-centric, round-to-nearest."""
    with torch.cuda.device(dh.device):
        M, H, dh1, dh3, a1, a3 = _silu_deriv(dh, h3, h1_raw)
        q1 = _quantize_with_amax(dh1, M, H, a1, True)
        q3 = _quantize_with_amax(dh3, M, H, a3, True)
        zero = torch.zeros(1, dtype=torch.float32, device=dh.device)
        amax_buf = torch.stack([a1[0], a3[0]])
        sync_buf = torch.zeros(4, dtype=torch.int32, device=dh.device)
    return (*q1, a1.narrow(0, 1, 1), zero, *q3, a3.narrow(0, 1, 1), zero.clone(), amax_buf, sync_buf, dh1, dh3)


def tk_silu_deriv_quantize_split_for_gemm_opt(dh, h3, h1_raw, return_transpose=True, encode_centric=True,
                                              data_stochastic_rounding=False, scale_stochastic_rounding=False,
                                              rht_axes="row", with_random_sign_mask=False, rng_seed=0,
                                              rng_subsequence=0, data_sr_axes="both"):
    """tk_quantize.cu:10063-10255 — 15-tuple: dh1 (row_fp4,row_sc,col_fp4,col_sc,row_sg,col_sg), dh3
    likewise, amaxes[4], dh1 bf16, dh3 bf16.  Built: round-to-nearest without Hadamard transform
    (``rht_axes="none"``); the stochastic-rounding and RHT variants raise until they are built."""
    if data_stochastic_rounding or scale_stochastic_rounding:
        raise RuntimeError("tk_silu_deriv_quantize_split_for_gemm_opt: stochastic rounding is not built yet")
    if rht_axes not in ("none", "", None):
        raise RuntimeError("tk_silu_deriv_quantize_split_for_gemm_opt: rht_axes other than 'none' is not built yet")
    with torch.cuda.device(dh.device):
        M, H, dh1, dh3, a1, a3 = _silu_deriv(dh, h3, h1_raw)
        q1 = _quantize_with_amax(dh1, M, H, a1, encode_centric, return_transpose)
        q3 = _quantize_with_amax(dh3, M, H, a3, encode_centric, return_transpose)
        amaxes = torch.stack([a1[0], a1[0], a3[0], a3[0]])
    sg1, sg3 = a1.narrow(0, 1, 1), a3.narrow(0, 1, 1)
    return (*q1, sg1, sg1, *q3, sg3, sg3, amaxes, dh1, dh3)
