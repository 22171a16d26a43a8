"""Host-side mirror of the reference's ``_tk_quant_v5`` extension module (NVFP4 producers).

Same function names, argument order, defaults, return tuples and error behaviour
(``RuntimeError`` on a rejected argument) as the pybind module defined at
fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:10815-11153.  Outputs are allocated with
torch on the input's device, kernels are enqueued on torch's current stream of that device
through the C ABI in ``include/fp4b200.h``.  There is no fallback path.
"""
from __future__ import annotations

import contextlib
import threading

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


def tk_quantize_nhsd_wo_for_gemm(input, return_transpose, encode_centric=True):
    """tk_quantize.cu:3006-3134 — attention output bf16 [B, H, S, 64] quantised as the matrix [B*S, H*64] that the
    output projection consumes, without a transposing copy; same 8-tuple as ``tk_quantize_for_gemm``."""
    if not isinstance(input, torch.Tensor) or not input.is_cuda or not input.is_contiguous():
        raise RuntimeError("input must be a contiguous CUDA tensor")
    if input.dtype != torch.bfloat16 or input.dim() != 4:
        raise RuntimeError("input must be bf16 [B, H, S, D]")
    B, H, S, D = (int(v) for v in input.shape)
    if D != 64:
        raise RuntimeError("NHSD WO direct quantization currently requires head_dim == 64")
    if S % 128:
        raise RuntimeError("NHSD WO direct quantization requires sequence length to be a multiple of 128")
    M, K = B * S, H * D
    if M % 128 or K % 128:
        raise RuntimeError("logical [B*S, H*D] dimensions must be multiples of 128")
    with torch.cuda.device(input.device):
        row_fp4, row_sc, col_fp4, col_sc = _alloc_operands(M, K, input.device, return_transpose)
        amax_sg = torch.empty(2, dtype=torch.float32, device=input.device)
        sync_buf = torch.zeros(4, dtype=torch.int32, device=input.device)
        _lib.call("fp4b200_nvfp4_quantize_nhsd_wo", input.data_ptr(), B, H, S, D, int(bool(return_transpose)),
                  int(bool(encode_centric)), row_fp4.data_ptr(), row_sc.data_ptr(),
                  _p(col_fp4) if return_transpose else None, _p(col_sc) if return_transpose else None,
                  amax_sg.data_ptr(), _stream(input))
    sg = amax_sg.narrow(0, 1, 1)
    return (row_fp4.view(_FP4), row_sc.view(_E4M3), col_fp4.view(_FP4) if return_transpose else col_fp4,
            col_sc.view(_E4M3) if return_transpose else col_sc, sg, sg, amax_sg, sync_buf)


def tk_group_quantize_dim1_split3_for_gemm(input0, input1, input2, data_stochastic_rounding=False, rng_seed=0,
                                           rng_subsequence=0, data_sr_axes="both"):
    """tk_quantize.cu:6425-6835 — three gradient streams [M, n_g] (the attention side's dQ, dK, dV), each quantised
    with its own tensor amax (encode-centric, round-to-nearest) straight into the column slices of one row-wise code
    matrix [M, N/2] and the row blocks of one column-wise code matrix [N, M/2], N = n_0 + n_1 + n_2.  Returns the
    reference's 15-tuple: (row code views, row scales, sg [3], column code views, column scales, full row codes,
    row scales concatenated along the block dimension, full column codes, column scales concatenated, three empty
    descriptor / barrier tensors' places, amax [3], ...).  Stochastic rounding on both axes takes the reference's
    default route (:6485-6548): one launch of the tuned kernel per stream, the streams at three consecutive
    invocation offsets; rounding one axis only (the reference's grouped kernel) is not built."""
    sr = bool(data_stochastic_rounding)
    if sr and _norm_sr_axes(data_sr_axes) != "both":
        raise RuntimeError("tk_group_quantize_dim1_split3_for_gemm: stochastic rounding of one axis only is not built")
    inputs = [input0, input1, input2]
    for t in inputs:
        if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise RuntimeError("split3 inputs must be CUDA bf16 matrices contiguous along the inner dimension")
        if t.device != input0.device:
            raise RuntimeError("split3 inputs must be on the same CUDA device")
    M = int(input0.shape[0])
    if any(int(t.shape[0]) != M for t in inputs):
        raise RuntimeError("split3 inputs must share the same row count")
    splits = [int(t.shape[1]) for t in inputs]
    n_total = sum(splits)
    if M % 128 or any(n % 128 for n in splits):
        raise RuntimeError("M and every split width must be multiples of 128")
    dev = input0.device
    u8 = dict(dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        fp4_row_full = torch.empty((M, n_total // 2), **u8)
        fp4_col_full = torch.empty((n_total, M // 2), **u8)
        xs = [t if t.is_contiguous() else t.contiguous() for t in inputs]   # the amax pass reads dense buffers
        sc_row = [torch.empty((M // 128, n // 64, 512), **u8) for n in splits]
        if sr:
            amax_sg = torch.empty((3, 2), dtype=torch.float32, device=dev)
            sc_col = [torch.empty((n // 128, M // 64, 512), **u8) for n in splits]
            off = 0
            for g, (x, n) in enumerate(zip(xs, splits)):
                _lib.call("fp4b200_nvfp4_amax", x.data_ptr(), M * n, amax_sg[g].data_ptr(), _stream(input0))
                state = _reserve_sr(input0, rng_seed, rng_subsequence, True)
                _lib.call("fp4b200_nvfp4_quantize_opt_into", x.data_ptr(), None, None, M, n, amax_sg[g].data_ptr(),
                          amax_sg[g].data_ptr(), 1, 1, 0, 0, 0, 0, 0, 1, 0, 0, 0, state.data_ptr(), 0,
                          fp4_row_full.data_ptr() + off // 2,
                          n_total // 2, sc_row[g].data_ptr(), fp4_col_full.data_ptr() + off * (M // 2),
                          sc_col[g].data_ptr(), None, _stream(input0))
                off += n
            sg_per_group = amax_sg[:, 1].contiguous()
            amax_tensor = amax_sg[:, 0].contiguous()
            sc_col_cat = torch.cat(sc_col, 0)
        else:
            # one amax launch and one quantiser launch for the three streams; the column-wise scales are written
            # where their concatenation holds them, so the per-stream tensors are its row blocks
            amax_pair = torch.empty((2, 3), dtype=torch.float32, device=dev)
            amax_tensor, sg_per_group = amax_pair[0], amax_pair[1]
            sc_col_cat = torch.empty((n_total // 128, M // 64, 512), **u8)
            _lib.call("fp4b200_nvfp4_quantize_split3_into", xs[0].data_ptr(), xs[1].data_ptr(), xs[2].data_ptr(), M,
                      splits[0], splits[1], splits[2], fp4_row_full.data_ptr(), sc_row[0].data_ptr(),
                      sc_row[1].data_ptr(), sc_row[2].data_ptr(), fp4_col_full.data_ptr(), sc_col_cat.data_ptr(),
                      amax_tensor.data_ptr(), sg_per_group.data_ptr(), _stream(input0))
            sc_col, off = [], 0
            for n in splits:
                sc_col.append(sc_col_cat.narrow(0, off // 128, n // 128))
                off += n
        fp4_row_list, fp4_col_list = [], []
        off = 0
        for n in splits:
            fp4_row_list.append(fp4_row_full.narrow(1, off // 2, n // 2))
            fp4_col_list.append(fp4_col_full.narrow(0, off, n).view(_FP4))
            off += n
        sc_row_cat = torch.cat(sc_row, 1).view(_E4M3)
        sc_col_cat = sc_col_cat.view(_E4M3)
        empty_u8 = torch.empty(0, **u8)
        empty_i32 = torch.empty(0, dtype=torch.int32, device=dev)
    return ([t for t in fp4_row_list], [t.view(_E4M3) for t in sc_row], sg_per_group, fp4_col_list,
            [t.view(_E4M3) for t in sc_col], fp4_row_full.view(_FP4), sc_row_cat, fp4_col_full.view(_FP4), sc_col_cat,
            empty_u8, torch.empty(0, dtype=torch.uint8), torch.empty(0, dtype=torch.int64, device=dev), amax_tensor,
            torch.zeros(6, dtype=torch.int32, device=dev), empty_i32)


def tk_group_quantize_dim1_for_gemm(input, col_split_sections):
    """tk_quantize.cu:6192-6416 — the column groups of ONE matrix [M, sum(sections)] (the concatenated dQ | dK | dV the
    reference falls back to when its split3 entry point is absent, tk_gemm.py:6020-6024), each quantised with its own
    tensor amax (encode-centric, round to nearest) into the column slices / row blocks of one pair of code matrices.
    Returns the reference's 9-tuple: (row code views, row scales, sg [G], column code views, column scales, full row
    codes, row scales concatenated, full column codes, column scales concatenated).  Three groups take the grouped
    launch of the split3 quantiser; other counts one quantiser call per group."""
    M, n_total = _check_bf16_2d(input, "input")
    sections = [int(v) for v in col_split_sections]
    if not sections or any(v <= 0 or v % 128 for v in sections) or sum(sections) != n_total:
        raise RuntimeError("column sections must be positive multiples of 128 that add up to the input's width")
    if len(sections) > 8:
        raise RuntimeError("Max 8 groups")
    parts, off = [], 0
    for n in sections:
        parts.append(input.narrow(1, off, n))
        off += n
    if len(sections) == 3:
        return tk_group_quantize_dim1_split3_for_gemm(*parts)[:9]
    dev = input.device
    u8 = dict(dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        fp4_row_full = torch.empty((M, n_total // 2), **u8)
        fp4_col_full = torch.empty((n_total, M // 2), **u8)
        sc_col_cat = torch.empty((n_total // 128, M // 64, 512), **u8)
        amax_sg = torch.empty((len(sections), 2), dtype=torch.float32, device=dev)
        sc_row, sc_col, rows, cols, off = [], [], [], [], 0
        for g, (t, n) in enumerate(zip(parts, sections)):
            x = t.contiguous()                                   # the amax pass reads a dense buffer
            sc_row.append(torch.empty((M // 128, n // 64, 512), **u8))
            sc_col.append(sc_col_cat.narrow(0, off // 128, n // 128))
            _lib.call("fp4b200_nvfp4_quantize_for_gemm_into", x.data_ptr(), M, n, 1, 1, fp4_row_full.data_ptr() + off // 2,
                      n_total // 2, sc_row[g].data_ptr(), fp4_col_full.data_ptr() + off * (M // 2), sc_col[g].data_ptr(),
                      amax_sg[g].data_ptr(), _stream(input))
            rows.append(fp4_row_full.narrow(1, off // 2, n // 2))
            cols.append(fp4_col_full.narrow(0, off, n).view(_FP4))
            off += n
        sc_row_cat = torch.cat(sc_row, 1).view(_E4M3)
    return (rows, [t.view(_E4M3) for t in sc_row], amax_sg[:, 1].contiguous(), cols, [t.view(_E4M3) for t in sc_col],
            fp4_row_full.view(_FP4), sc_row_cat, fp4_col_full.view(_FP4), sc_col_cat.view(_E4M3))


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


def row_rms_reduce(row_rms_partial, hidden_size, epsilon):
    """inv_rms [M] from GEMM-epilogue row partials [M, P] (kernel: common/c1_rms_reduce.cuh:11-38)."""
    p = row_rms_partial
    if (not isinstance(p, torch.Tensor) or not p.is_cuda or p.dtype != torch.float32 or p.dim() != 2
            or not p.is_contiguous()):
        raise RuntimeError("row_rms_partial must be contiguous CUDA float32 [M,P]")
    inv_rms = torch.empty(p.shape[0], dtype=torch.float32, device=p.device)
    with torch.cuda.device(p.device):
        _lib.call("fp4b200_row_rms_reduce", p.data_ptr(), p.shape[0], p.shape[1], int(hidden_size), float(epsilon),
                  inv_rms.data_ptr(), _stream(p))
    return inv_rms


def tk_fused_norm_quantize_from_row_rms_partial(input, gamma, row_rms_partial, epsilon, with_silu, return_transpose):
    """tk_quantize.cu:8266-8308 — inverse RMS from per-32-column partial sums of squares [M, K/32] left by a
    GEMM epilogue, then the fused producer with that inverse RMS."""
    M, K = _check_bf16_2d(input, "input")
    if K > 4096:
        raise RuntimeError("row_rms_partial warp reducer supports K <= 4096")
    if (not isinstance(row_rms_partial, torch.Tensor) or row_rms_partial.dim() != 2
            or tuple(row_rms_partial.shape) != (M, K // 32) or row_rms_partial.device != input.device):
        raise RuntimeError("row_rms_partial shape must be [M,K/32] on the input device")
    inv_rms = row_rms_reduce(row_rms_partial, K, epsilon)
    return _fused_norm_impl(input, gamma, 0.0, with_silu, return_transpose, inv_rms)


def tk_batched_quantize_for_gemm(inputs, return_transpose, encode_centric=True):
    """tk_quantize.cu:11117-11152 — tk_quantize_for_gemm over a list; returns eight lists
    (row_fp4s, row_scs, col_fp4s, col_scs, sgs, sgs, amax_keepalive, sync_keepalive)."""
    outs = [tk_quantize_for_gemm(x, return_transpose, encode_centric) for x in inputs]
    return tuple([o[i] for o in outs] for i in range(8))


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


# ---- allocate-once / launch-many pairs (CUDA-graph capture) --------------------------------------
# The *_launch functions run into buffers made by their *_alloc twin and allocate nothing, so they can be
# captured into a CUDA graph.  The library keeps a few KB of device scratch per (device, stream), created on
# a stream's first call: run one call on the capture stream before capturing.

def tk_v4_quantize_for_gemm_alloc(M, K, return_transpose, device):
    """tk_quantize.cu:3622-3641 — (row_fp4, row_sc, col_fp4, col_sc, amax_buf, sync_buf), codes and scales as uint8."""
    if M % 128 or K % 128:
        raise RuntimeError("M and K must be multiples of 128")
    dev = torch.device(device)
    row_fp4, row_sc, col_fp4, col_sc = _alloc_operands(int(M), int(K), dev, bool(return_transpose))
    return (row_fp4, row_sc, col_fp4, col_sc, torch.empty(2, dtype=torch.float32, device=dev),
            torch.empty(4, dtype=torch.int32, device=dev))


def tk_v4_quantize_for_gemm_launch(input, return_transpose, encode_centric, row_fp4, row_sc, col_fp4, col_sc, amax_buf,
                                   sync_buf):
    """tk_quantize.cu:3646-3799 — amax + row/column quantisation into the caller's buffers; returns
    (row_fp4, row_sc, col_fp4, col_sc, sg, sg) as views of them."""
    M, K = _check_bf16_2d(input, "input")
    if row_fp4.numel() != M * K // 2 or row_sc.numel() != M * K // 16 or amax_buf.numel() < 2:
        raise RuntimeError("buffers do not match the input shape (use tk_v4_quantize_for_gemm_alloc)")
    if return_transpose and (col_fp4.numel() != M * K // 2 or col_sc.numel() != M * K // 16):
        raise RuntimeError("return_transpose needs the column buffers of tk_v4_quantize_for_gemm_alloc(..., True, ...)")
    with torch.cuda.device(input.device):
        _lib.call("fp4b200_nvfp4_quantize_for_gemm", input.data_ptr(), M, K, int(bool(return_transpose)),
                  int(bool(encode_centric)), row_fp4.data_ptr(), row_sc.data_ptr(),
                  col_fp4.data_ptr() if return_transpose else None, col_sc.data_ptr() if return_transpose else None,
                  amax_buf.data_ptr(), _stream(input))
    sg = amax_buf.narrow(0, 1, 1)
    return (row_fp4.view(_FP4), row_sc.view(_E4M3), col_fp4.view(_FP4) if return_transpose else col_fp4,
            col_sc.view(_E4M3) if return_transpose else col_sc, sg, sg)


def tk_silu_deriv_quantize_split_for_gemm_alloc(M, H, device):
    """tk_quantize.cu:9660-9690 — 14 buffers: operands of dh1 (4), of dh3 (4), sg_buf [2], zero_buf [1], amax_buf [2],
    sync_buf [4], dh1, dh3 (bf16 [M, H])."""
    if M % 128 or H % 128:
        raise RuntimeError("M and H must be multiples of 128")
    dev = torch.device(device)
    o1 = _alloc_operands(int(M), int(H), dev, True)
    o2 = _alloc_operands(int(M), int(H), dev, True)
    f32 = dict(dtype=torch.float32, device=dev)
    return (o1[0].view(_FP4), o1[1].view(_E4M3), o1[2].view(_FP4), o1[3].view(_E4M3),
            o2[0].view(_FP4), o2[1].view(_E4M3), o2[2].view(_FP4), o2[3].view(_E4M3),
            torch.empty(2, **f32), torch.zeros(1, **f32), torch.empty(2, **f32),
            torch.empty(4, dtype=torch.int32, device=dev),
            torch.empty((int(M), int(H)), dtype=torch.bfloat16, device=dev),
            torch.empty((int(M), int(H)), dtype=torch.bfloat16, device=dev))


def tk_silu_deriv_quantize_split_for_gemm_launch(dh, h3, h1_raw, out1_fp4, out1_sc, out1_fp4_t, out1_sc_t, out2_fp4,
                                                 out2_sc, out2_fp4_t, out2_sc_t, sg_buf, zero_buf, amax_buf, sync_buf, dh1,
                                                 dh3):
    """tk_quantize.cu:9696-9887 — SiLU-derivative producer (encode-centric, round-to-nearest) into the caller's
    buffers; returns the 12-tuple (dh1 operands, sg1, zero, dh3 operands, sg3, zero).  amax_buf receives the two
    tensor maxima; sync_buf (unused by this implementation's kernels) carries them between the launches."""
    M, H = _check_bf16_2d(dh, "dh")
    _same_shape_bf16(dh, h3, h1_raw)
    for t in (dh1, dh3):
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or tuple(t.shape) != (M, H):
            raise RuntimeError("dh1 / dh3 must be contiguous bf16 [M, H]")
    if sg_buf.numel() < 2 or amax_buf.numel() < 2 or sync_buf.numel() < 4 or sync_buf.dtype != torch.int32:
        raise RuntimeError("sg_buf [2], amax_buf [2] and int32 sync_buf [4] are required")
    for t in (out1_fp4, out1_fp4_t, out2_fp4, out2_fp4_t):
        if t.numel() * t.element_size() != M * H // 2:
            raise RuntimeError("code buffers do not match the input shape")
    for t in (out1_sc, out1_sc_t, out2_sc, out2_sc_t):
        if t.numel() != M * H // 16:
            raise RuntimeError("scale buffers do not match the input shape")
    with torch.cuda.device(dh.device):
        st = _stream(dh)
        pair = sync_buf.view(torch.float32)          # [amax1, sg1, amax3, sg3] between the launches
        _lib.call("fp4b200_silu_deriv_bf16", dh.data_ptr(), h3.data_ptr(), h1_raw.data_ptr(), dh.numel(), dh1.data_ptr(),
                  dh3.data_ptr(), pair.data_ptr(), pair.data_ptr() + 8, st)
        for x, amax_ptr, slot, (c, s_, ct, st_) in ((dh1, pair.data_ptr(), 0, (out1_fp4, out1_sc, out1_fp4_t, out1_sc_t)),
                                                     (dh3, pair.data_ptr() + 8, 1, (out2_fp4, out2_sc, out2_fp4_t, out2_sc_t))):
            _lib.call("fp4b200_nvfp4_quantize", x.data_ptr(), M, H, amax_ptr, None, 1, c.data_ptr(), s_.data_ptr(),
                      ct.data_ptr(), st_.data_ptr(), sg_buf.data_ptr() + 4 * slot, st)
        amax_buf.narrow(0, 0, 1).copy_(pair.narrow(0, 0, 1))
        amax_buf.narrow(0, 1, 1).copy_(pair.narrow(0, 2, 1))
    return (out1_fp4, out1_sc, out1_fp4_t, out1_sc_t, sg_buf.narrow(0, 0, 1), zero_buf,
            out2_fp4, out2_sc, out2_fp4_t, out2_sc_t, sg_buf.narrow(0, 1, 1), zero_buf)


# ---- stochastic rounding / Hadamard ("opt") producers -----------------------------------------

_U64 = (1 << 64) - 1
_SR_STRIDE = 1 << 32   # counter distance between two stochastic launches (tk_quantize.cu:443)


def tk_sr_invocation_count(device=None) -> int:
    """Number of stochastic-rounding launches reserved so far on ``device`` in this process: launch n draws at the
    Philox offset ``rng_subsequence + n * 2**32``.  The counter lives on the device, as the reference's
    (tk_sr_invocation_offset, tk_quantize.cu:443-481); reading it waits for the current stream."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        out = torch.empty(1, dtype=torch.int64, device=dev)
        _lib.call("fp4b200_sr_get_invocation_offset", out.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
        return (int(out.item()) & _U64) >> 32


def tk_set_sr_invocation_count(n: int, device=None) -> None:
    """Restores the counter (checkpoint resume, tests) in stream order; no counterpart in the reference, whose
    counter cannot be set."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _lib.call("fp4b200_sr_set_invocation_offset", (int(n) * _SR_STRIDE) & _U64,
                  torch.cuda.current_stream(dev).cuda_stream)


_PRODUCER_STATE = threading.local()


@contextlib.contextmanager
def producer_sr_state(state):
    """Inside the block, the stochastic quantisers of this module called from this thread number their launches from
    ``state`` — a producer's persistent int64[2] {seed, next subsequence} on its device, e.g. a row of
    ``localcta_sr_state.LocalCTASRState`` — instead of the device-wide counter: each call takes the pair as its Philox
    key and base and advances ``state[1]`` by 2**32 per launch it makes, on its own stream; the ``rng_seed`` /
    ``rng_subsequence`` arguments are ignored.  ``None`` leaves the device-wide numbering in force (the calling
    convention of get_localcta_sr_state, which returns None without an installed table)."""
    if state is not None and (not isinstance(state, torch.Tensor) or not state.is_cuda or state.dtype != torch.int64
                              or state.numel() != 2 or not state.is_contiguous()):
        raise RuntimeError("producer_sr_state: the state must be a contiguous CUDA int64 tensor with two elements")
    before = getattr(_PRODUCER_STATE, "state", None)
    _PRODUCER_STATE.state = state
    try:
        yield
    finally:
        _PRODUCER_STATE.state = before


def _reserve_sr(t, rng_seed, rng_subsequence, use_sr, launches=1):
    """Device words {key, base} for the next ``launches`` stochastic launches on t's device (None without
    stochastic rounding): a one-thread kernel advances the device counter, so a captured graph reserves new
    numbers on every replay (tk_make_advancing_rng_state, tk_quantize.cu:469-481).  Launch k of the group passes
    the relative offset ``k * 2**32``.  Under producer_sr_state the numbers come from that producer's own pair."""
    if not use_sr:
        return None
    state = torch.empty(2, dtype=torch.int64, device=t.device)
    own = getattr(_PRODUCER_STATE, "state", None)
    if own is not None:
        if own.device != t.device:
            raise RuntimeError(f"producer_sr_state: the state is on {own.device}, its producer's input on {t.device}")
        _lib.call("fp4b200_sr_reserve_from_state", own.data_ptr(), state.data_ptr(), int(launches), _stream(t))
        return state
    _lib.call("fp4b200_sr_prepare_state", state.data_ptr(), int(rng_seed) & _U64, int(rng_subsequence) & _U64,
              int(launches), _stream(t))
    return state


def _norm_axes(rht_axes):
    a = str(rht_axes).lower().replace("-", "_")
    if a not in ("none", "row", "col", "both", "rowcol", "row_col"):
        raise RuntimeError(f"Unsupported regular TK RHT axes: {rht_axes}")
    return a in ("row", "both", "rowcol", "row_col"), a in ("col", "both", "rowcol", "row_col")


def _norm_sr_axes(data_sr_axes):
    a = str(data_sr_axes).lower().replace("-", "_")
    a = {"all": "both", "rowcol": "both", "row_col": "both", "column": "col", "columns": "col", "wgrad": "col",
         "dgrad": "row", "off": "none", "0": "none"}.get(a, a)
    if a not in ("none", "row", "col", "both"):
        raise RuntimeError(f"Unsupported regular TK data SR axes: {data_sr_axes}")
    return a


def _amax_plain(x):
    amax_sg = torch.empty(2, dtype=torch.float32, device=x.device)
    _lib.call("fp4b200_nvfp4_amax", x.data_ptr(), x.numel(), amax_sg.data_ptr(), _stream(x))
    return amax_sg


def _amax_rht(x, along_k, sign, seed, subseq, gamma=None, inv_rms=None, with_plain=False):
    """Tensor amax / sg of the 16-point transform of x; ``with_plain`` (scan along M only): also x's own amax / sg
    from the same read, returned second."""
    M, K = x.shape
    amax_sg = torch.empty(2, dtype=torch.float32, device=x.device)
    plain = torch.empty(2, dtype=torch.float32, device=x.device) if with_plain else None
    _lib.call("fp4b200_nvfp4_rht16_amax", x.data_ptr(), _p(gamma), _p(inv_rms), M, K, int(along_k), int(sign),
              int(seed) & _U64, int(subseq) & _U64, amax_sg.data_ptr(), _p(plain), _stream(x))
    return (amax_sg, plain) if with_plain else amax_sg


def _launch_opt(x, amax_row, amax_col, return_transpose, sr, encode_centric, row_rht, col_rht, return_row, seed, offset,
                sign, sign_seed, sign_subseq, gamma=None, inv_rms=None, sr_mode=None, offset_col=0, scale_sr=False,
                rng_state=None, out=None):
    """One launch, the counterpart of tk_quantize_transpose (tk_quantize.cu:3807-3926).  ``sr_mode`` 2 / 3:
    stochastic rounding on the row pass only (the bytes of the reference's row-only launch at ``offset``) /
    on the column pass only (at ``offset_col``), the other pass rounded to nearest in the same launch."""
    M, K = x.shape
    u8 = dict(dtype=torch.uint8, device=x.device)
    if out is not None:      # the caller's buffers (alloc / launch pairs)
        row_fp4, row_sc, col_fp4, col_sc = out
    else:
        row_fp4 = torch.empty((M, K // 2), **u8) if return_row else None
        row_sc = torch.empty((M // 128, K // 64, 512), **u8) if return_row else None
        col_fp4 = torch.empty((K, M // 2), **u8) if return_transpose else None
        col_sc = torch.empty((K // 128, M // 64, 512), **u8) if return_transpose else None
    # encode-centric scale SR: scratch for the map of blocks that draw no scale word (the reference thread's later
    # draws move up behind such a block, quantize_transpose_tuned.cuh:244-254)
    zero_map = torch.empty(M * K // 32, **u8) if (scale_sr and encode_centric) else None
    _lib.call("fp4b200_nvfp4_quantize_opt", x.data_ptr(), _p(gamma), _p(inv_rms), M, K, amax_row.data_ptr(),
              amax_col.data_ptr(), int(bool(encode_centric)), int(bool(sr)) if sr_mode is None else int(sr_mode),
              int(bool(row_rht)), int(bool(col_rht)),
              int(bool(sign)), int(sign_seed) & _U64, int(sign_subseq) & _U64, int(bool(return_row)),
              int(seed) & _U64, int(offset) & _U64, int(offset_col) & _U64, _p(rng_state), int(bool(scale_sr)), _p(row_fp4), _p(row_sc),
              _p(col_fp4), _p(col_sc), _p(zero_map), _stream(x))
    return row_fp4, row_sc, col_fp4, col_sc


def tk_quantize_transpose(input, amax_row, amax_col, return_transpose, stochastic_rounding=False, encode_centric=True,
                          scale_stochastic_rounding=False, row_rht=False, col_rht=False, return_row=True, rng_state=None):
    """tk_quantize.cu:3807-3926 — quantise with pre-computed device amaxes; ``rng_state`` = int64[2] tensor
    ``[seed, offset]``.  Returns (row_fp4, row_sc, col_fp4, col_sc) as uint8 tensors."""
    _check_bf16_2d(input, "input")
    state = None
    if stochastic_rounding or scale_stochastic_rounding:
        if (rng_state is None or rng_state.numel() < 2 or rng_state.dtype != torch.int64 or not rng_state.is_contiguous()
                or rng_state.device != input.device):
            raise RuntimeError("rng_state must be a contiguous int64[2] tensor [seed, offset] on the input's device "
                               "with stochastic rounding")
        state = rng_state   # read by the kernel, as in the reference: no host round trip
    with torch.cuda.device(input.device):
        out = _launch_opt(input, amax_row, amax_col, return_transpose, stochastic_rounding, encode_centric, row_rht,
                          col_rht, return_row, 0, 0, False, 0, 0, scale_sr=scale_stochastic_rounding, rng_state=state)
    # shapes as the reference returns them: scale bytes as [rows, blocks per row] (the bytes are in the GEMM's tile order)
    M, K = input.shape
    # With return_row = False the reference still returns row tensors of full shape that nothing has written; so here.
    u8 = dict(dtype=torch.uint8, device=input.device)
    rf, rs, cf, cs = out
    return (torch.empty((M, K // 2), **u8) if rf is None else rf, torch.empty((M, K // 16), **u8) if rs is None else rs.view(M, K // 16),
            torch.empty((0,), **u8) if cf is None else cf, torch.empty((0,), **u8) if cs is None else cs.view(K, M // 16))


def tk_quantize_for_gemm_opt(input, return_transpose=True, encode_centric=True, data_stochastic_rounding=False,
                             scale_stochastic_rounding=False, rht_axes="none", with_random_sign_mask=False, rng_seed=0,
                             rng_subsequence=0, global_scale_target=448.0, data_sr_axes="both"):
    """tk_quantize.cu:4299-4540 — returns (row_fp4, row_sc, col_fp4, col_sc, row_sg, col_sg).  Same choice of
    amaxes, number of launches and Philox offsets as the reference."""
    M, K = _check_bf16_2d(input, "input")
    scale_sr = bool(scale_stochastic_rounding)
    if not (0.0 < float(global_scale_target) <= 512.0):
        raise RuntimeError(f"global_scale_target must be finite and in (0, 512], got {global_scale_target}")
    row_rht, col_rht = _norm_axes(rht_axes)
    if float(global_scale_target) != 448.0 and (row_rht or col_rht):
        raise RuntimeError("non-default global_scale_target is currently supported only with rht_axes='none'")
    axes = _norm_sr_axes(data_sr_axes)
    row_sr = bool(data_stochastic_rounding) and axes in ("row", "both")
    col_sr = bool(data_stochastic_rounding) and axes in ("col", "both")
    if not (row_rht or col_rht or row_sr or col_sr or scale_sr) and float(global_scale_target) == 448.0:
        base = tk_quantize_for_gemm(input, return_transpose, encode_centric)
        return base[:6]
    use_sr = row_sr or col_sr or scale_sr
    sign = bool(with_random_sign_mask)
    with torch.cuda.device(input.device):
        if row_rht:
            row_amax = _amax_rht(input, True, sign, rng_seed, rng_subsequence)
            col_amax = _amax_rht(input, False, sign, rng_seed, rng_subsequence) if col_rht else _amax_plain(input)
        elif col_rht:
            # the column operand's scan yields the untransformed maximum for the row operand from the same read
            col_amax, row_amax = _amax_rht(input, False, sign, rng_seed, rng_subsequence, with_plain=True)
        else:
            col_amax = row_amax = _amax_plain(input)
            if float(global_scale_target) != 448.0:
                row_amax.mul_(448.0 / float(global_scale_target))
        row_mat, col_mat = row_rht and sign, col_rht and sign     # the reference materialises these
        if return_transpose and (row_mat or col_mat) and not (scale_sr and not (row_sr or col_sr)):
            # the reference runs a row launch and a column launch over a sign-flipped, transformed copy; the sign
            # flip happens inside this library's transform, so one launch reads the input once and gives each pass
            # the stream of its reference launch
            state = _reserve_sr(input, rng_seed, rng_subsequence, use_sr, 2)
            mode = 0 if not (row_sr or col_sr) else (4 if (row_sr and col_sr) else (2 if row_sr else 3))
            rf, rs, cf, cs = _launch_opt(input, row_amax, col_amax, True, row_sr or col_sr, encode_centric, row_rht, col_rht,
                                         True, rng_seed, 0, sign, rng_seed, rng_subsequence, sr_mode=mode,
                                         offset_col=_SR_STRIDE, scale_sr=scale_sr, rng_state=state)
        elif return_transpose and not row_mat and row_sr == col_sr and not col_mat:
            state = _reserve_sr(input, rng_seed, rng_subsequence, use_sr)
            rf, rs, cf, cs = _launch_opt(input, row_amax, col_amax, True, row_sr, encode_centric, row_rht, col_rht,
                                         True, rng_seed, 0, sign, rng_seed, rng_subsequence, scale_sr=scale_sr,
                                         rng_state=state)
        elif return_transpose and not row_mat and not col_mat:
            # the reference serves "one axis stochastic" with a row launch and a column launch, each taking
            # an offset; here one launch reads the input once and produces the same bytes
            state = _reserve_sr(input, rng_seed, rng_subsequence, use_sr, 2)
            rf, rs, cf, cs = _launch_opt(input, row_amax, col_amax, True, True, encode_centric, row_rht, col_rht, True,
                                         rng_seed, 0, sign, rng_seed, rng_subsequence, sr_mode=2 if row_sr else 3,
                                         offset_col=_SR_STRIDE, scale_sr=scale_sr, rng_state=state)
        else:
            state = _reserve_sr(input, rng_seed, rng_subsequence, use_sr)
            rf, rs, _, _ = _launch_opt(input, row_amax, row_amax, False, row_sr, encode_centric, row_rht, False, True,
                                       rng_seed, 0, sign, rng_seed, rng_subsequence, scale_sr=scale_sr, rng_state=state)
            cf = cs = None
            if return_transpose:
                state = _reserve_sr(input, rng_seed, rng_subsequence, use_sr)
                _, _, cf, cs = _launch_opt(input, col_amax, col_amax, True, col_sr, encode_centric, False, col_rht,
                                           False, rng_seed, 0, sign, rng_seed, rng_subsequence, scale_sr=scale_sr,
                                           rng_state=state)
    empty = torch.empty((0,), dtype=torch.uint8, device=input.device)
    row_sg = row_amax.narrow(0, 1, 1)
    col_sg = col_amax.narrow(0, 1, 1) if return_transpose else row_sg
    return (rf.view(_FP4), rs.view(_E4M3), cf.view(_FP4) if cf is not None else empty,
            cs.view(_E4M3) if cs is not None else empty, row_sg, col_sg)


def tk_fused_norm_quantize_opt(input, gamma, epsilon, return_transpose=True, encode_centric=True,
                               data_stochastic_rounding=False, scale_stochastic_rounding=False, rht_axes="row",
                               with_random_sign_mask=False, rng_seed=0, rng_subsequence=0):
    """tk_quantize.cu:8465-8586 — fused RMSNorm + row-Hadamard (+ stochastic rounding) quantisation; returns
    (row_fp4, row_sc, col_fp4, col_sc, row_sg, col_sg, inv_rms).  As in the reference only the row transform
    without sign mask is accepted."""
    M, K = _check_bf16_2d(input, "input")
    row_rht, col_rht = _norm_axes(rht_axes)
    if not row_rht or col_rht:
        raise RuntimeError("tk_fused_norm_quantize_opt currently supports the regular-TK QKV row-RHT contract only")
    if with_random_sign_mask:
        raise RuntimeError("tk_fused_norm_quantize_opt does not yet fuse random-sign RHT")
    if gamma.dtype != torch.bfloat16 or gamma.numel() != K or not gamma.is_contiguous() or gamma.device != input.device:
        raise RuntimeError("gamma must be contiguous CUDA bfloat16 [K] on the input device")
    sr = bool(data_stochastic_rounding)
    scale_sr = bool(scale_stochastic_rounding)
    with torch.cuda.device(input.device):
        inv_rms = torch.empty(M, dtype=torch.float32, device=input.device)
        col_amax = torch.empty(2, dtype=torch.float32, device=input.device)
        # inverse RMS in the summation order of this producer's own kernel, then the tensor maximum with it
        _lib.call("fp4b200_nvfp4_rmsnorm_inv_rms_opt", input.data_ptr(), gamma.data_ptr(), float(epsilon), M, K,
                  inv_rms.data_ptr(), _stream(input))
        _lib.call("fp4b200_nvfp4_rmsnorm_stats", input.data_ptr(), gamma.data_ptr(), float(epsilon), M, K,
                  inv_rms.data_ptr(), 0, col_amax.data_ptr(), _stream(input))
        row_amax = _amax_rht(input, True, False, 0, 0, gamma, inv_rms)
        state = _reserve_sr(input, rng_seed, rng_subsequence, sr or scale_sr)
        rf, rs, cf, cs = _launch_opt(input, row_amax, col_amax, True, sr, encode_centric, True, False, True, rng_seed,
                                     0, False, 0, 0, gamma, inv_rms, scale_sr=scale_sr, rng_state=state)
    return (rf.view(_FP4), rs.view(_E4M3), cf.view(_FP4), cs.view(_E4M3), row_amax.narrow(0, 1, 1),
            col_amax.narrow(0, 1, 1), inv_rms)


def tk_silu_deriv_quantize_split_for_gemm_opt(dh, h3, h1_raw, return_transpose=True, encode_centric=True,
                                              data_stochastic_rounding=False, scale_stochastic_rounding=False,
                                              rht_axes="row", with_random_sign_mask=False, rng_seed=0,
                                              rng_subsequence=0, data_sr_axes="both"):
    """tk_quantize.cu:10063-10255 — 15-tuple: dh1 (row_fp4,row_sc,col_fp4,col_sc,row_sg,col_sg), dh3 likewise,
    amaxes[4], dh1 bf16, dh3 bf16.  As in the reference the row operand is Hadamard-transformed
    (``rht_axes="row"``), there is no sign mask, and each of dh1/dh3 takes one Philox offset shared by its
    row and column launches (also when only the scale bytes round stochastically); ``rht_axes="none"`` is
    accepted as an extension (no transform)."""
    if not return_transpose:
        raise RuntimeError("split2 opt producer currently requires return_transpose=True")
    row_rht, col_rht = _norm_axes(rht_axes)
    if col_rht:
        raise RuntimeError(f"split2 opt producer currently supports the row-RHT regular-TK contract only; got {rht_axes}")
    if with_random_sign_mask:
        raise RuntimeError("split2 opt producer does not support random RHT sign masks yet")
    scale_sr = bool(scale_stochastic_rounding)
    axes = _norm_sr_axes(data_sr_axes)
    row_sr = bool(data_stochastic_rounding) and axes in ("row", "both")
    col_sr = bool(data_stochastic_rounding) and axes in ("col", "both")
    use_sr = row_sr or col_sr or scale_sr
    with torch.cuda.device(dh.device):
        M, H, dh1, dh3, a1, a3 = _silu_deriv(dh, h3, h1_raw)
        outs, sgs, amax_list = [], [], []
        for t, orig in ((dh1, a1), (dh3, a3)):
            row_amax = _amax_rht(t, True, False, 0, 0) if row_rht else orig
            state = _reserve_sr(t, rng_seed, rng_subsequence, use_sr)
            if row_sr == col_sr:
                q = _launch_opt(t, row_amax, orig, True, row_sr, encode_centric, row_rht, False, True, rng_seed, 0,
                                False, 0, 0, scale_sr=scale_sr, rng_state=state)
            else:
                # one axis stochastic: the reference's row launch and column launch (same offset) as one
                q = _launch_opt(t, row_amax, orig, True, True, encode_centric, row_rht, False, True, rng_seed, 0,
                                False, 0, 0, sr_mode=2 if row_sr else 3, offset_col=0, scale_sr=scale_sr,
                                rng_state=state)
            outs.append((q[0].view(_FP4), q[1].view(_E4M3), q[2].view(_FP4), q[3].view(_E4M3)))
            sgs.append((row_amax.narrow(0, 1, 1), orig.narrow(0, 1, 1)))
            amax_list += [row_amax[0], orig[0]]
        amaxes = torch.stack(amax_list)
    return (*outs[0], *sgs[0], *outs[1], *sgs[1], amaxes, dh1, dh3)


def tk_silu_deriv_quantize_split_for_gemm_opt_alloc(M, H, device):
    """tk_quantize.cu:10259-10290 — the 11 buffers of the pair: operands of dh1 (4) and of dh3 (4) as uint8, sgs [4],
    amaxes [4], sync_buf [4].  Call outside graph capture."""
    if M % 128 or H % 128:
        raise RuntimeError("M and H must be multiples of 128")
    dev = torch.device(device)
    o1 = _alloc_operands(int(M), int(H), dev, True)
    o2 = _alloc_operands(int(M), int(H), dev, True)
    f32 = dict(dtype=torch.float32, device=dev)
    return (*o1, *o2, torch.empty(4, **f32), torch.empty(4, **f32), torch.empty(4, dtype=torch.int32, device=dev))


def tk_silu_deriv_quantize_split_for_gemm_opt_launch(dh, h3, h1_raw, return_transpose, encode_centric,
                                                     data_stochastic_rounding, scale_stochastic_rounding, rht_axes,
                                                     with_random_sign_mask, rng_seed, rng_subsequence, out1_fp4, out1_sc,
                                                     out1_fp4_t, out1_sc_t, out2_fp4, out2_sc, out2_fp4_t, out2_sc_t, sgs,
                                                     amaxes, sync_buf, data_sr_axes="both"):
    """tk_quantize.cu:10292-10388 — the SiLU-derivative producer with the row operand Hadamard-transformed and
    optional stochastic rounding, into the caller's buffers; safe to capture in a CUDA graph (the launch number
    comes from the device counter).  Returns the 12-tuple (dh1 operands, row sg, column sg, dh3 operands, row sg,
    column sg); amaxes receives [row amax 1, column amax 1, row amax 3, column amax 3].

    Random stream, as in the reference's kernel for this pair (persistent_silu_deriv_quantize.cuh:64-74,150-176): ONE
    reserved launch number; dh1 and dh3 each draw from that same offset, in the order of a single launch of the
    tuned quantiser with both passes (row blocks, then column blocks of each 64 x 64 stage).  That order exists here
    for rounding both axes, or neither, stochastically; one axis alone is not built for this pair.  dh1 and dh3 in
    bf16 are temporaries from torch's allocator (the reference keeps them in shared memory)."""
    M, H = _check_bf16_2d(dh, "dh")
    _same_shape_bf16(dh, h3, h1_raw)
    if not return_transpose:
        raise RuntimeError("split2 opt prealloc producer currently requires return_transpose=True")
    row_rht, col_rht = _norm_axes(rht_axes)
    if not row_rht or col_rht:
        raise RuntimeError(f"split2 opt prealloc producer currently supports the row-RHT regular-TK contract only; got {rht_axes}")
    if with_random_sign_mask:
        raise RuntimeError("split2 opt prealloc producer does not support random RHT sign masks yet")
    axes = _norm_sr_axes(data_sr_axes)
    row_sr = bool(data_stochastic_rounding) and axes in ("row", "both")
    col_sr = bool(data_stochastic_rounding) and axes in ("col", "both")
    if row_sr != col_sr:
        raise RuntimeError("split2 opt prealloc producer: stochastic rounding of one axis only is not built")
    scale_sr = bool(scale_stochastic_rounding)
    if sgs.numel() < 4 or amaxes.numel() < 4 or sgs.dtype != torch.float32 or amaxes.dtype != torch.float32:
        raise RuntimeError("sgs [4] and amaxes [4] (float32) are required")
    if sync_buf.numel() < 4 or sync_buf.dtype != torch.int32:
        raise RuntimeError("int32 sync_buf [4] is required")
    outs = ((out1_fp4, out1_sc, out1_fp4_t, out1_sc_t), (out2_fp4, out2_sc, out2_fp4_t, out2_sc_t))
    for c, s_, ct, st_ in outs:
        if c.numel() * c.element_size() != M * H // 2 or ct.numel() * ct.element_size() != M * H // 2:
            raise RuntimeError("code buffers do not match the input shape")
        if s_.numel() != M * H // 16 or st_.numel() != M * H // 16:
            raise RuntimeError("scale buffers do not match the input shape")
    with torch.cuda.device(dh.device):
        _, _, dh1, dh3, a1, a3 = _silu_deriv(dh, h3, h1_raw)
        state = _reserve_sr(dh, rng_seed, rng_subsequence, row_sr or scale_sr)
        for g, (t, orig, out) in enumerate(((dh1, a1, outs[0]), (dh3, a3, outs[1]))):
            row_amax = _amax_rht(t, True, False, 0, 0)
            _launch_opt(t, row_amax, orig, True, row_sr, encode_centric, True, False, True, rng_seed, 0, False, 0, 0,
                        scale_sr=scale_sr, rng_state=state, out=out)
            amaxes.narrow(0, 2 * g, 1).copy_(row_amax.narrow(0, 0, 1))
            amaxes.narrow(0, 2 * g + 1, 1).copy_(orig.narrow(0, 0, 1))
            sgs.narrow(0, 2 * g, 1).copy_(row_amax.narrow(0, 1, 1))
            sgs.narrow(0, 2 * g + 1, 1).copy_(orig.narrow(0, 1, 1))
    return (out1_fp4.view(_FP4), out1_sc.view(_E4M3), out1_fp4_t.view(_FP4), out1_sc_t.view(_E4M3),
            sgs.narrow(0, 0, 1), sgs.narrow(0, 1, 1),
            out2_fp4.view(_FP4), out2_sc.view(_E4M3), out2_fp4_t.view(_FP4), out2_sc_t.view(_E4M3),
            sgs.narrow(0, 2, 1), sgs.narrow(0, 3, 1))
