"""Host-side mirror of the reference's ``mxfp4_quant_v4`` extension module (MXFP4 producers).

Names, argument order, defaults and return tuples follow the pybind module at
fp4_runtime/TK_quantisation/mxfp4_v4/tk_quantize.cu:7281-7724: codes ``[rows, cols/2]`` as
``float4_e2m1fn_x2``, E8M0 scale bytes ``[rows/128, cols/128, 32, 16]`` as uint8.  ``mode``: 0 RTE,
1 ceil ("encode", the production setting), 2 floor.  Dense FFN subset only.
"""
from __future__ import annotations

import os

import torch

from . import _lib
from .tk_quant_v5 import _check_bf16_2d, _same_shape_bf16, _stream

_FP4 = torch.float4_e2m1fn_x2


def _one_pass_act():
    """FP4B200_MX_ONE_PASS=0 routes the SwiGLU producers through the element kernel and a bf16 intermediate again
    (A/B runs; the bytes are the same)."""
    return os.environ.get("FP4B200_MX_ONE_PASS", "1") != "0"


def _alloc(M, K, device, want_col):
    u8 = dict(dtype=torch.uint8, device=device)
    row_fp4 = torch.empty((M, K // 2), **u8)
    row_sc = torch.empty((M // 128, K // 128, 32, 16), **u8)
    if not want_col:
        return row_fp4, row_sc, None, None
    return row_fp4, row_sc, torch.empty((K, M // 2), **u8), torch.empty((K // 128, M // 128, 32, 16), **u8)


def _quant(x, mode, want_col):
    M, K = _check_bf16_2d(x, "input")
    with torch.cuda.device(x.device):
        rf, rs, cf, cs = _alloc(M, K, x.device, want_col)
        _lib.call("fp4b200_mxfp4_quantize", x.data_ptr(), M, K, int(mode), rf.data_ptr(), rs.data_ptr(),
                  None if cf is None else cf.data_ptr(), None if cs is None else cs.data_ptr(), _stream(x))
    return rf, rs, cf, cs


def mxfp4_quantize_for_gemm(input, mode=0):
    """tk_quantize.cu:7282 — (fp4, scales), row-wise only."""
    rf, rs, _, _ = _quant(input, mode, False)
    return rf.view(_FP4), rs


def _row_sr(input, mode, data_sr, scale_sr, rht_block, sign, rng_seed, rng_subsequence):
    M, K = _check_bf16_2d(input, "input")
    with torch.cuda.device(input.device):
        rf, rs, _, _ = _alloc(M, K, input.device, False)
        _lib.call("fp4b200_mxfp4_quantize_row_sr", input.data_ptr(), M, K, int(mode), int(bool(data_sr)), int(bool(scale_sr)),
                  int(rht_block), int(bool(sign)), int(rng_seed) & 0xFFFFFFFFFFFFFFFF,
                  int(rng_subsequence) & 0xFFFFFFFFFFFFFFFF, rf.data_ptr(), rs.data_ptr(), _stream(input))
    return rf.view(_FP4), rs


def mxfp4_quantize_for_gemm_opt(input, mode=0, data_stochastic_rounding=False, scale_stochastic_rounding=False,
                                rng_seed=1234, rng_subsequence=0):
    """tk_quantize.cu:1848-1881 (bound at 7285) — row-wise (fp4, scales) with stochastic rounding of the codes
    and / or of the E8M0 scale bytes, on the reference's Philox stream for (rng_seed, rng_subsequence); with
    neither flag it is ``mxfp4_quantize_for_gemm``."""
    if not data_stochastic_rounding and not scale_stochastic_rounding:
        return mxfp4_quantize_for_gemm(input, mode)
    return _row_sr(input, mode, data_stochastic_rounding, scale_stochastic_rounding, 0, False, rng_seed, rng_subsequence)


def _check_rht_block(rht_block_size):
    if int(rht_block_size) not in (16, 32):
        raise RuntimeError("RHT block size must be 16 or 32")
    return int(rht_block_size)


def mxfp4_quantize_for_gemm_opt_rht(input, mode=0, data_stochastic_rounding=False, scale_stochastic_rounding=False,
                                    rht_block_size=16, with_random_sign_mask=True, rng_seed=1234, rng_subsequence=0):
    """tk_quantize.cu:1883-2060 (bound at 7292) — as ``mxfp4_quantize_for_gemm_opt`` behind a Hadamard transform of
    16 or 32 consecutive elements of each row (``with_random_sign_mask``: the reference's fixed sign diagonal in
    front of it); both rounding flags may be off."""
    return _row_sr(input, mode, data_stochastic_rounding, scale_stochastic_rounding, _check_rht_block(rht_block_size),
                   with_random_sign_mask, rng_seed, rng_subsequence)


# The reference advances a device-global offset by 2^40 per row + column launch that uses its generator
# (mxfp4_forward_sr_invocation_offset, tk_quantize.cu:33-48) and adds it to the caller's subsequence; the mirror
# keeps the count on the host, readable and settable so that a resumed run or a test can restore it.
_SR_INVOCATION_STRIDE = 1 << 40
_sr_invocations = 0


def mxfp4_forward_sr_invocation_count():
    return _sr_invocations


def mxfp4_set_forward_sr_invocation_count(n):
    global _sr_invocations
    _sr_invocations = int(n)


def _rowcol_sr(input, mode, data_sr, scale_sr, rht_block, sign, row_rht, col_rht, rng_seed, rng_subsequence):
    global _sr_invocations
    M, K = _check_bf16_2d(input, "input")
    base = int(rng_subsequence) & 0xFFFFFFFFFFFFFFFF
    if data_sr or scale_sr or (rht_block and sign):   # the launches that prepare a generator state (tk_quantize.cu:2853-2860)
        if torch.cuda.is_current_stream_capturing():
            # host-side launch number: a captured graph would replay one offset on every launch
            raise RuntimeError("stochastic rounding inside CUDA-graph capture would replay one Philox offset on every "
                               "graph launch: run the stochastic quantisers outside the captured region")
        base = (base + _sr_invocations * _SR_INVOCATION_STRIDE) & 0xFFFFFFFFFFFFFFFF
        _sr_invocations += 1
    with torch.cuda.device(input.device):
        rf, rs, cf, cs = _alloc(M, K, input.device, True)
        _lib.call("fp4b200_mxfp4_quantize_row_and_col_sr", input.data_ptr(), M, K, int(mode), int(bool(data_sr)),
                  int(bool(scale_sr)), int(rht_block), int(bool(sign)), int(bool(row_rht)), int(bool(col_rht)),
                  int(rng_seed) & 0xFFFFFFFFFFFFFFFF, base, rf.data_ptr(), rs.data_ptr(), cf.data_ptr(), cs.data_ptr(),
                  _stream(input))
    return rf.view(_FP4), rs, cf.view(_FP4), cs


def mxfp4_quantize_row_and_col_opt(input, mode=0, data_stochastic_rounding=False, scale_stochastic_rounding=False,
                                   rng_seed=1234, rng_subsequence=0):
    """tk_quantize.cu:2920-2953 (bound at 7397) — (row_fp4, row_sc, col_fp4, col_sc) with stochastic rounding; the
    codes of the two views agree element by element ("correlated" rounding).  With neither flag it is
    ``mxfp4_quantize_row_and_col``."""
    if not data_stochastic_rounding and not scale_stochastic_rounding:
        return mxfp4_quantize_row_and_col(input, mode)
    return _rowcol_sr(input, mode, data_stochastic_rounding, scale_stochastic_rounding, 0, False, False, False, rng_seed,
                      rng_subsequence)


def mxfp4_quantize_row_and_col_opt_rht(input, mode=0, data_stochastic_rounding=False, scale_stochastic_rounding=False,
                                       rht_block_size=16, with_random_sign_mask=True, rng_seed=1234, rng_subsequence=0):
    """tk_quantize.cu:3082-3102 (bound at 7404) — Hadamard transform along M on the column view only."""
    return _rowcol_sr(input, mode, data_stochastic_rounding, scale_stochastic_rounding, _check_rht_block(rht_block_size),
                      with_random_sign_mask, False, True, rng_seed, rng_subsequence)


def mxfp4_quantize_row_and_col_opt_rht_both(input, mode=0, data_stochastic_rounding=False,
                                            scale_stochastic_rounding=False, rht_block_size=16,
                                            with_random_sign_mask=True, rng_seed=1234, rng_subsequence=0):
    """tk_quantize.cu:3104-3124 (bound at 7413) — transform along K on the row view and along M on the column view."""
    return _rowcol_sr(input, mode, data_stochastic_rounding, scale_stochastic_rounding, _check_rht_block(rht_block_size),
                      with_random_sign_mask, True, True, rng_seed, rng_subsequence)


def mxfp4_quantize_row_and_col_opt_rht_row_only(input, mode=0, data_stochastic_rounding=False,
                                                scale_stochastic_rounding=False, rht_block_size=16,
                                                with_random_sign_mask=True, rng_seed=1234, rng_subsequence=0):
    """tk_quantize.cu:3126-3146 (bound at 7422) — transform along K on the row view only."""
    return _rowcol_sr(input, mode, data_stochastic_rounding, scale_stochastic_rounding, _check_rht_block(rht_block_size),
                      with_random_sign_mask, True, False, rng_seed, rng_subsequence)


def mxfp4_quantize_row_and_col(input, mode=0):
    """tk_quantize.cu:7344 — (row_fp4, row_sc, col_fp4, col_sc)."""
    rf, rs, cf, cs = _quant(input, mode, True)
    return rf.view(_FP4), rs, cf.view(_FP4), cs


def mxfp4_fused_rmsnorm_quantize_row_and_col(input, norm_weight, epsilon, mode=0):
    """tk_quantize.cu:7701 — (row_fp4, row_sc, col_fp4, col_sc, inv_rms)."""
    M, K = _check_bf16_2d(input, "input")
    if (not isinstance(norm_weight, torch.Tensor) or norm_weight.dtype != torch.bfloat16 or norm_weight.numel() != K
            or not norm_weight.is_contiguous() or norm_weight.device != input.device):
        raise RuntimeError("norm_weight must be contiguous CUDA bfloat16 [K] on the input device")
    with torch.cuda.device(input.device):
        rf, rs, cf, cs = _alloc(M, K, input.device, True)
        inv_rms = torch.empty(M, dtype=torch.float32, device=input.device)
        st = _stream(input)
        # inverse RMS only (MXFP4 has no tensor scale), in this producer's own summation order
        _lib.call("fp4b200_mxfp4_rmsnorm_inv_rms", input.data_ptr(), norm_weight.data_ptr(), float(epsilon), M, K,
                  inv_rms.data_ptr(), st)
        _lib.call("fp4b200_mxfp4_quantize_normed", input.data_ptr(), norm_weight.data_ptr(), inv_rms.data_ptr(), M, K,
                  int(mode), rf.data_ptr(), rs.data_ptr(), cf.data_ptr(), cs.data_ptr(), st)
    return rf.view(_FP4), rs, cf.view(_FP4), cs, inv_rms


def mxfp4_fused_silu_mul_quantize_row_and_col(h1_raw, h3, mode=0):
    """tk_quantize.cu:7435 — (row_fp4, row_sc, col_fp4, col_sc) of ``bf16(silu(h1_raw) * h3)``."""
    M, H = _check_bf16_2d(h1_raw, "h1_raw")
    _same_shape_bf16(h1_raw, h3)
    with torch.cuda.device(h1_raw.device):
        if _one_pass_act():
            rf, rs, cf, cs = _alloc(M, H, h1_raw.device, True)
            _lib.call("fp4b200_mxfp4_silu_mul_quantize", h1_raw.data_ptr(), h3.data_ptr(), M, H, int(mode), rf.data_ptr(),
                      rs.data_ptr(), cf.data_ptr(), cs.data_ptr(), _stream(h1_raw))
            return rf.view(_FP4), rs, cf.view(_FP4), cs
        h = torch.empty_like(h1_raw)
        amax_sg = torch.empty(2, dtype=torch.float32, device=h1_raw.device)
        _lib.call("fp4b200_silu_mul_bf16", h1_raw.data_ptr(), h3.data_ptr(), h1_raw.numel(), h.data_ptr(),
                  amax_sg.data_ptr(), _stream(h1_raw))
    return mxfp4_quantize_row_and_col(h, mode)


def mxfp4_quantize_weight_2d(input):
    """tk_quantize.cu:2734-2737 — one E8M0 scale per 32x32 tile shared by both orientations;
    (row_fp4, row_sc, col_fp4, col_sc)."""
    N, K = _check_bf16_2d(input, "input")
    with torch.cuda.device(input.device):
        rf, rs, cf, cs = _alloc(N, K, input.device, True)
        _lib.call("fp4b200_mxfp4_quantize_weight_2d", input.data_ptr(), N, K, rf.data_ptr(), rs.data_ptr(),
                  cf.data_ptr(), cs.data_ptr(), _stream(input))
    return rf.view(_FP4), rs, cf.view(_FP4), cs


def mxfp4_fused_rmsnorm_quantize_row_and_col_from_row_rms_partial(input, norm_weight, row_rms_partial, epsilon, mode=1):
    """tk_quantize.cu:6960-7052 — inverse RMS from GEMM-epilogue row partials [M, K/256], then the fused
    RMSNorm + row/col quantiser; (row_fp4, row_sc, col_fp4, col_sc, inv_rms).  The reference accepts only
    mode 1 ("encode"), K == 4096 and M % 256 == 0 here; so does this mirror."""
    from .tk_quant_v5 import row_rms_reduce
    M, K = _check_bf16_2d(input, "input")
    if int(mode) != 1:
        raise RuntimeError("MXFP4 exact C/D/E production path requires encode mode")
    if M % 256 or K != 4096:
        raise RuntimeError("MXFP4 exact C/D/E consumer requires [M,4096] with M divisible by 256")
    if (not isinstance(norm_weight, torch.Tensor) or norm_weight.dtype != torch.bfloat16 or norm_weight.numel() != K
            or not norm_weight.is_contiguous() or norm_weight.device != input.device):
        raise RuntimeError("norm_weight must be contiguous CUDA bfloat16 [K] on the input device")
    if tuple(row_rms_partial.shape) != (M, K // 256) or row_rms_partial.device != input.device:
        raise RuntimeError("row_rms_partial shape must be [M,K/256]")
    inv_rms = row_rms_reduce(row_rms_partial, K, epsilon)
    with torch.cuda.device(input.device):
        rf, rs, cf, cs = _alloc(M, K, input.device, True)
        _lib.call("fp4b200_mxfp4_quantize_normed", input.data_ptr(), norm_weight.data_ptr(), inv_rms.data_ptr(), M, K,
                  1, rf.data_ptr(), rs.data_ptr(), cf.data_ptr(), cs.data_ptr(), _stream(input))
    return rf.view(_FP4), rs, cf.view(_FP4), cs, inv_rms



def mxfp4_fused_silu_deriv_quantize_split2_row_and_col(dh, h3, h1_raw, mode=0):
    """tk_quantize.cu:4513-4620 — ``dh1 = bf16(dh*h3*silu'(h1_raw))``, ``dh3 = bf16(dh*silu(h1_raw))``, each
    quantised row- and column-wise; outputs stacked on a leading dimension of 2 (dh1 first):
    (row_fp4 [2,M,H/2], row_sc [2,M/128,H/128,32,16], col_fp4 [2,H,M/2], col_sc [2,H/128,M/128,32,16])."""
    from .tk_quant_v5 import tk_silu_deriv_split_bf16
    M, H = _check_bf16_2d(dh, "dh")
    _same_shape_bf16(dh, h3, h1_raw)
    u8 = dict(dtype=torch.uint8, device=dh.device)
    row_fp4 = torch.empty((2, M, H // 2), **u8)
    row_sc = torch.empty((2, M // 128, H // 128, 32, 16), **u8)
    col_fp4 = torch.empty((2, H, M // 2), **u8)
    col_sc = torch.empty((2, H // 128, M // 128, 32, 16), **u8)
    if _one_pass_act():
        with torch.cuda.device(dh.device):
            _lib.call("fp4b200_mxfp4_silu_deriv_quantize_split2", dh.data_ptr(), h3.data_ptr(), h1_raw.data_ptr(), M, H,
                      int(mode), row_fp4.data_ptr(), row_sc.data_ptr(), col_fp4.data_ptr(), col_sc.data_ptr(), _stream(dh))
        return row_fp4.view(_FP4), row_sc, col_fp4.view(_FP4), col_sc
    dh1, dh3 = tk_silu_deriv_split_bf16(dh, h3, h1_raw)
    with torch.cuda.device(dh.device):
        for i, t in enumerate((dh1, dh3)):
            _lib.call("fp4b200_mxfp4_quantize", t.data_ptr(), M, H, int(mode), row_fp4[i].data_ptr(), row_sc[i].data_ptr(),
                      col_fp4[i].data_ptr(), col_sc[i].data_ptr(), _stream(dh))
    return row_fp4.view(_FP4), row_sc, col_fp4.view(_FP4), col_sc


def mxfp4_quantize_col_only(input, mode=0):
    """tk_quantize.cu:2404-2470 — the column-wise operand alone (the wgrad's view of a tensor whose row-wise operand
    nobody reads): (col_fp4 [K, M/2], col_sc [K/128, M/128, 32, 16])."""
    M, K = _check_bf16_2d(input, "input")
    u8 = dict(dtype=torch.uint8, device=input.device)
    col_fp4, col_sc = torch.empty((K, M // 2), **u8), torch.empty((K // 128, M // 128, 32, 16), **u8)
    with torch.cuda.device(input.device):
        _lib.call("fp4b200_mxfp4_quantize", input.data_ptr(), M, K, int(mode), None, None, col_fp4.data_ptr(),
                  col_sc.data_ptr(), _stream(input))
    return col_fp4.view(_FP4), col_sc


def mxfp4_quantize_nhsd_wo_row_and_col(input, mode=0):
    """tk_quantize.cu:2739-2830 — the attention output ``input`` [B, H, S, D] quantised as the [B*S, H*D] matrix the
    output projection consumes, without the transposing copy; returns (row_fp4 [M, K/2], row_sc [M/128, K/128, 32, 16],
    col_fp4 [K, M/2], col_sc [K/128, M/128, 32, 16])."""
    if not isinstance(input, torch.Tensor) or not input.is_cuda or not input.is_contiguous():
        raise RuntimeError("NHSD WO MXFP4 quantize expects a contiguous CUDA tensor")
    if input.dtype != torch.bfloat16 or input.dim() != 4:
        raise RuntimeError("NHSD WO MXFP4 quantize expects bf16 [B,H,S,D]")
    B, H, S, D = (int(v) for v in input.shape)
    if D % 64:
        raise RuntimeError("NHSD WO MXFP4 quantize requires head_dim to be a multiple of 64")
    if S % 128:
        raise RuntimeError("NHSD WO MXFP4 quantize requires sequence length to be a multiple of 128")
    M, K = B * S, H * D
    if M % 128 or K % 128:
        raise RuntimeError("logical [B*S,H*D] dimensions must be multiples of 128")
    u8 = dict(dtype=torch.uint8, device=input.device)
    row_fp4, row_sc = torch.empty((M, K // 2), **u8), torch.empty((M // 128, K // 128, 32, 16), **u8)
    col_fp4, col_sc = torch.empty((K, M // 2), **u8), torch.empty((K // 128, M // 128, 32, 16), **u8)
    with torch.cuda.device(input.device):
        _lib.call("fp4b200_mxfp4_quantize_nhsd_wo", input.data_ptr(), B, H, S, D, int(mode), row_fp4.data_ptr(),
                  row_sc.data_ptr(), col_fp4.data_ptr(), col_sc.data_ptr(), _stream(input))
    return row_fp4.view(_FP4), row_sc, col_fp4.view(_FP4), col_sc


def _quantize_split(inputs, outs, mode):
    import ctypes
    M = None
    for t in inputs:
        if (not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous() or t.dtype != torch.bfloat16
                or t.dim() != 2 or t.shape[0] % 128 or t.shape[1] % 128):
            raise RuntimeError("split inputs must be contiguous bf16 matrices with dims divisible by 128")
        if M is not None and int(t.shape[0]) != M:
            raise RuntimeError("split inputs must have the same M dimension")
        M = int(t.shape[0])
    K = sum(int(t.shape[1]) for t in inputs)
    if outs is None:
        u8 = dict(dtype=torch.uint8, device=inputs[0].device)
        outs = (torch.empty((M, K // 2), **u8).view(_FP4), torch.empty((M // 128, K // 128, 32, 16), **u8),
                torch.empty((K, M // 2), **u8).view(_FP4), torch.empty((K // 128, M // 128, 32, 16), **u8))
    else:
        _check_operand_outs(*outs, M, K)
    n = len(inputs)
    xs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in inputs])
    widths = (ctypes.c_int64 * n)(*[int(t.shape[1]) for t in inputs])
    with torch.cuda.device(inputs[0].device):
        _lib.call("fp4b200_mxfp4_quantize_split", xs, widths, n, M, int(mode), outs[0].data_ptr(), outs[1].data_ptr(),
                  outs[2].data_ptr(), outs[3].data_ptr(), _stream(inputs[0]))
    return outs


def mxfp4_quantize_split2_row_and_col(input0, input1, mode=0):
    """tk_quantize.cu:5375-5440 — the operands of ``cat([input0, input1], dim=1)`` without the bf16 concatenation
    (dh1 | dh3 of a fused gate/up projection): (row_fp4 [M, K/2], row_sc [M/128, K/128, 32, 16], col_fp4 [K, M/2],
    col_sc [K/128, M/128, 32, 16]), K = K0 + K1."""
    return _quantize_split((input0, input1), None, mode)


def mxfp4_quantize_split2_row_and_col_launch_inplace(input0, input1, row_fp4, row_sc, col_fp4, col_sc, mode=0):
    """tk_quantize.cu:5443-5470 — the same into the caller's tensors; returns None."""
    _quantize_split((input0, input1), (row_fp4, row_sc, col_fp4, col_sc), mode)


def mxfp4_quantize_split3_row_and_col(input0, input1, input2, mode=0):
    """tk_quantize.cu:6254-6345 — the operands of ``cat([input0, input1, input2], dim=1)`` without the concatenation
    (dQ | dK | dV on the way to the QKV dgrad and wgrad); shapes as the two-input form with K = K0 + K1 + K2."""
    return _quantize_split((input0, input1, input2), None, mode)


def mxfp4_quantize_split3_row_and_col_launch_inplace(input0, input1, input2, row_fp4, row_sc, col_fp4, col_sc, mode=0):
    """tk_quantize.cu:6348-6440 — the same into the caller's tensors; returns None."""
    _quantize_split((input0, input1, input2), (row_fp4, row_sc, col_fp4, col_sc), mode)


def mxfp4_quantize_split3_row_and_col_inverse_rope_live64(input0, input1, input2, rope_cs, rope_seq_len, mode=0):
    """tk_quantize.cu:6551-6644 — ``mxfp4_quantize_split3_row_and_col`` with the inverse rotary embedding of the first two
    inputs (dQ, dK; heads of 64, neighbouring columns paired) folded into the load; ``rope_cs`` fp32
    [rope_seq_len, 32, 2], ``rope_seq_len`` a power of two."""
    inputs = (input0, input1, input2)
    M = None
    for t in inputs:
        if (not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous() or t.dtype != torch.bfloat16
                or t.dim() != 2 or t.shape[0] % 128 or t.shape[1] % 128):
            raise RuntimeError("split inputs must be contiguous bf16 matrices with dims divisible by 128")
        if M is not None and int(t.shape[0]) != M:
            raise RuntimeError("split inputs must have the same M dimension")
        M = int(t.shape[0])
    seq = int(rope_seq_len)
    if seq <= 0 or seq & (seq - 1):
        raise RuntimeError("rope_seq_len must be a positive power of two")
    if (not isinstance(rope_cs, torch.Tensor) or not rope_cs.is_cuda or not rope_cs.is_contiguous()
            or rope_cs.dtype != torch.float32 or tuple(rope_cs.shape) != (seq, 32, 2)):
        raise RuntimeError("rope_cs must have shape (rope_seq_len, 32, 2)")
    ks = [int(t.shape[1]) for t in inputs]
    K = sum(ks)
    u8 = dict(dtype=torch.uint8, device=input0.device)
    row_fp4, row_sc = torch.empty((M, K // 2), **u8), torch.empty((M // 128, K // 128, 32, 16), **u8)
    col_fp4, col_sc = torch.empty((K, M // 2), **u8), torch.empty((K // 128, M // 128, 32, 16), **u8)
    with torch.cuda.device(input0.device):
        _lib.call("fp4b200_mxfp4_quantize_split3_inverse_rope", input0.data_ptr(), input1.data_ptr(), input2.data_ptr(), M,
                  ks[0], ks[1], ks[2], rope_cs.data_ptr(), seq, int(mode), row_fp4.data_ptr(), row_sc.data_ptr(),
                  col_fp4.data_ptr(), col_sc.data_ptr(), _stream(input0))
    return row_fp4.view(_FP4), row_sc, col_fp4.view(_FP4), col_sc


def mxfp4_fused_silu_mul_quantize_row_and_col_strided(h13, H, h3_offset, mode=0):
    """tk_quantize.cu:4105-4132 — ``bf16(silu(h1) * h3)`` quantised row- and column-wise, h1 and h3 read out of the
    packed gate|up activation ``h13`` [M, stride] (h1 in columns [0, H), h3 in [h3_offset, h3_offset + H)); returns
    (row_fp4 [M, H/2], row_sc [M/128, H/128, 32, 16], col_fp4 [H, M/2], col_sc [H/128, M/128, 32, 16])."""
    if not isinstance(h13, torch.Tensor) or not h13.is_cuda or not h13.is_contiguous() or h13.dtype != torch.bfloat16 or h13.dim() != 2:
        raise RuntimeError("h13 must be a contiguous 2-D CUDA bf16 tensor")
    M, H, h3_offset = int(h13.shape[0]), int(H), int(h3_offset)
    if M % 128 or H % 128:
        raise RuntimeError("M and H must be multiples of 128")
    if h3_offset < H or h3_offset + H > int(h13.shape[1]):
        raise RuntimeError("h13 must contain packed h1 and h3 slices")
    u8 = dict(dtype=torch.uint8, device=h13.device)
    row_fp4, row_sc = torch.empty((M, H // 2), **u8), torch.empty((M // 128, H // 128, 32, 16), **u8)
    col_fp4, col_sc = torch.empty((H, M // 2), **u8), torch.empty((H // 128, M // 128, 32, 16), **u8)
    with torch.cuda.device(h13.device):
        _lib.call("fp4b200_mxfp4_silu_mul_quantize_strided", h13.data_ptr(), int(h13.shape[1]), h3_offset, M, H, int(mode),
                  row_fp4.data_ptr(), row_sc.data_ptr(), col_fp4.data_ptr(), col_sc.data_ptr(), _stream(h13))
    return row_fp4.view(_FP4), row_sc, col_fp4.view(_FP4), col_sc


def mxfp4_fused_silu_deriv_quantize_split2_row_and_col_strided_combined(dh, h13, H, h3_offset, mode=0):
    """tk_quantize.cu:5015-5099 — the two gradients of the packed gate|up activation ``h13`` [M, stride] (h1 in columns
    [0, H), h3 in [h3_offset, h3_offset + H)) laid out for the one-pass split dgrad GEMM: (row_fp4 [M, H] = dh1's
    codes | dh3's, row_sc [M/128, 2H/128, 32, 16] = dh1's tiles | dh3's per row block, col_fp4 [2H, M/2] and col_sc
    [2H/128, M/128, 32, 16] = dh1's over dh3's).  ``dh`` may be wider than H (its first H columns are read)."""
    for t, n in ((dh, "dh"), (h13, "h13")):
        if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous() or t.dtype != torch.bfloat16 or t.dim() != 2:
            raise RuntimeError(f"{n} must be a contiguous 2-D CUDA bf16 tensor")
    M, H, h3_offset = int(dh.shape[0]), int(H), int(h3_offset)
    if int(h13.shape[0]) != M:
        raise RuntimeError("dh and h13 row count mismatch")
    if M % 128 or H % 128:
        raise RuntimeError("M and H must be divisible by 128")
    if int(dh.shape[1]) < H:
        raise RuntimeError("dh stride must cover H")
    if h3_offset < H or h3_offset + H > int(h13.shape[1]):
        raise RuntimeError("h13 must contain packed h1 and h3 slices")
    u8 = dict(dtype=torch.uint8, device=dh.device)
    row_fp4 = torch.empty((M, H), **u8)
    row_sc = torch.empty((M // 128, 2 * H // 128, 32, 16), **u8)
    col_fp4 = torch.empty((2 * H, M // 2), **u8)
    col_sc = torch.empty((2 * H // 128, M // 128, 32, 16), **u8)
    with torch.cuda.device(dh.device):
        _lib.call("fp4b200_mxfp4_silu_deriv_quantize_split2_combined", dh.data_ptr(), int(dh.shape[1]), h13.data_ptr(),
                  int(h13.shape[1]), h3_offset, M, H, int(mode), row_fp4.data_ptr(), row_sc.data_ptr(), col_fp4.data_ptr(),
                  col_sc.data_ptr(), _stream(dh))
    return row_fp4.view(_FP4), row_sc, col_fp4.view(_FP4), col_sc


def mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols(dh, h3, h1_raw, mode=0):
    """tk_quantize.cu:4708-4810 — dh1 and dh3 with the row-wise operand in the one-pass split dgrad GEMM's layout and
    the column-wise operands apart: (row_fp4 [M, H] = dh1's codes | dh3's, row_sc [M/128, 2H/128, 32, 16],
    col0_fp4 [H, M/2], col0_sc [H/128, M/128, 32, 16], col1_fp4, col1_sc)."""
    M, H = _check_bf16_2d(dh, "dh")
    _same_shape_bf16(dh, h3, h1_raw)
    u8 = dict(dtype=torch.uint8, device=dh.device)
    row_fp4 = torch.empty((M, H), **u8).view(_FP4)
    row_sc = torch.empty((M // 128, 2 * H // 128, 32, 16), **u8)
    cols = [torch.empty((H, M // 2), **u8).view(_FP4) for _ in range(2)]
    col_scs = [torch.empty((H // 128, M // 128, 32, 16), **u8) for _ in range(2)]
    mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols_launch_inplace(dh, h3, h1_raw, row_fp4, row_sc, cols[0],
                                                                                col_scs[0], cols[1], col_scs[1], mode)
    return row_fp4, row_sc, cols[0], col_scs[0], cols[1], col_scs[1]


def mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols_launch_inplace(dh, h3, h1_raw, row_fp4, row_sc, col0_fp4,
                                                                                col0_sc, col1_fp4, col1_sc, mode=0):
    """tk_quantize.cu:4813-4905 — the same into the caller's tensors; returns None."""
    M, H = _check_bf16_2d(dh, "dh")
    _same_shape_bf16(dh, h3, h1_raw)
    _check_out(row_fp4, (M, H), True, "row_fp4")
    _check_out(row_sc, (M // 128, 2 * H // 128, 32, 16), False, "row_sc")
    for t, n in ((col0_fp4, "col0_fp4"), (col1_fp4, "col1_fp4")):
        _check_out(t, (H, M // 2), True, n)
    for t, n in ((col0_sc, "col0_sc"), (col1_sc, "col1_sc")):
        _check_out(t, (H // 128, M // 128, 32, 16), False, n)
    with torch.cuda.device(dh.device):
        _lib.call("fp4b200_mxfp4_silu_deriv_quantize_split2_splitcols", dh.data_ptr(), h3.data_ptr(), h1_raw.data_ptr(), M, H,
                  int(mode), row_fp4.data_ptr(), row_sc.data_ptr(), col0_fp4.data_ptr(), col0_sc.data_ptr(),
                  col1_fp4.data_ptr(), col1_sc.data_ptr(), _stream(dh))


# ---- *_launch_inplace twins: the caller owns the outputs -----------------------------------------

def _check_out(t, shape, fp4, name):
    want = _FP4 if fp4 else torch.uint8
    if (not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous() or t.dtype != want
            or tuple(t.shape) != tuple(shape)):
        raise RuntimeError(f"{name} must be a contiguous CUDA {'float4_e2m1fn_x2' if fp4 else 'uint8'} tensor of shape "
                           f"{tuple(shape)}")


def _check_operand_outs(row_fp4, row_sc, col_fp4, col_sc, M, K, lead=()):
    _check_out(row_fp4, (*lead, M, K // 2), True, "row_fp4")
    _check_out(row_sc, (*lead, M // 128, K // 128, 32, 16), False, "row_sc")
    _check_out(col_fp4, (*lead, K, M // 2), True, "col_fp4")
    _check_out(col_sc, (*lead, K // 128, M // 128, 32, 16), False, "col_sc")


def mxfp4_quantize_row_and_col_launch_inplace(input, row_fp4, row_sc, col_fp4, col_sc, mode=0):
    """tk_quantize.cu:3149-3229 — row and column quantisation into the caller's tensors; returns None."""
    M, K = _check_bf16_2d(input, "input")
    _check_operand_outs(row_fp4, row_sc, col_fp4, col_sc, M, K)
    with torch.cuda.device(input.device):
        _lib.call("fp4b200_mxfp4_quantize", input.data_ptr(), M, K, int(mode), row_fp4.data_ptr(), row_sc.data_ptr(),
                  col_fp4.data_ptr(), col_sc.data_ptr(), _stream(input))


def mxfp4_fused_silu_mul_quantize_row_and_col_launch_inplace(h1_raw, h3, row_fp4, row_sc, col_fp4, col_sc, mode=0):
    """tk_quantize.cu:3231-3310 — operands of ``bf16(silu(h1_raw) * h3)`` into the caller's tensors; returns None.
    One pass: the product lives in shared memory only, as in the reference."""
    M, H = _check_bf16_2d(h1_raw, "h1_raw")
    _same_shape_bf16(h1_raw, h3)
    _check_operand_outs(row_fp4, row_sc, col_fp4, col_sc, M, H)
    with torch.cuda.device(h1_raw.device):
        if _one_pass_act():
            _lib.call("fp4b200_mxfp4_silu_mul_quantize", h1_raw.data_ptr(), h3.data_ptr(), M, H, int(mode),
                      row_fp4.data_ptr(), row_sc.data_ptr(), col_fp4.data_ptr(), col_sc.data_ptr(), _stream(h1_raw))
            return
        h = torch.empty_like(h1_raw)
        amax_sg = torch.empty(2, dtype=torch.float32, device=h1_raw.device)
        st = _stream(h1_raw)
        _lib.call("fp4b200_silu_mul_bf16", h1_raw.data_ptr(), h3.data_ptr(), h1_raw.numel(), h.data_ptr(),
                  amax_sg.data_ptr(), st)
        _lib.call("fp4b200_mxfp4_quantize", h.data_ptr(), M, H, int(mode), row_fp4.data_ptr(), row_sc.data_ptr(),
                  col_fp4.data_ptr(), col_sc.data_ptr(), st)


def mxfp4_fused_silu_deriv_quantize_split2_row_and_col_launch_inplace(dh, h3, h1_raw, row_fp4, row_sc, col_fp4, col_sc,
                                                                      mode=0):
    """tk_quantize.cu:4611-4700 — the stacked operands of dh1 and dh3 (leading dimension 2) into the caller's
    tensors; returns None."""
    from .tk_quant_v5 import tk_silu_deriv_split_bf16
    M, H = _check_bf16_2d(dh, "dh")
    _same_shape_bf16(dh, h3, h1_raw)
    _check_operand_outs(row_fp4, row_sc, col_fp4, col_sc, M, H, lead=(2,))
    if _one_pass_act():
        with torch.cuda.device(dh.device):
            _lib.call("fp4b200_mxfp4_silu_deriv_quantize_split2", dh.data_ptr(), h3.data_ptr(), h1_raw.data_ptr(), M, H,
                      int(mode), row_fp4.data_ptr(), row_sc.data_ptr(), col_fp4.data_ptr(), col_sc.data_ptr(), _stream(dh))
        return
    dh1, dh3 = tk_silu_deriv_split_bf16(dh, h3, h1_raw)
    with torch.cuda.device(dh.device):
        for i, t in enumerate((dh1, dh3)):
            _lib.call("fp4b200_mxfp4_quantize", t.data_ptr(), M, H, int(mode), row_fp4[i].data_ptr(), row_sc[i].data_ptr(),
                      col_fp4[i].data_ptr(), col_sc[i].data_ptr(), _stream(dh))
