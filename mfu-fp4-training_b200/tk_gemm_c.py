"""Host-side mirror of the reference's ``_C`` extension module (NVFP4 tcgen05 GEMMs).

Same names and argument order as the pybind module at
fp4_runtime/ThunderKittens/kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:2851-3034: operands are
packed ``[rows, K/2]`` code tensors, scales ``[rows/128, K/64, 512]`` (or any contiguous view of
the same bytes), tensor scales fp32 ``[1]`` on the device; ``D`` is pre-allocated bf16 and written
in place; every function returns ``None``.  Kernels go to torch's current stream.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib


def _chk_operand(t, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
        raise RuntimeError(f"{name} must be a contiguous CUDA tensor")
    if t.element_size() != 1:
        raise RuntimeError(f"{name} must be a 1-byte dtype (packed fp4 / fp8 scale bytes)")


def _shapes(A, B, D_cols_total=None):
    if A.dim() != 2 or B.dim() != 2:
        raise RuntimeError("A and B must be 2-D packed tensors [rows, K/2]")
    M, Kh = A.shape
    N, Kh2 = B.shape
    if Kh != Kh2:
        raise RuntimeError(f"K mismatch between A ({2 * Kh}) and B ({2 * Kh2})")
    return M, N, 2 * Kh


def _chk_sg(t, name, n=1):
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.float32 or t.numel() < n:
        raise RuntimeError(f"{name} must be a CUDA float32 tensor with at least {n} element(s)")


def _chk_out(D, M, N, dtype=torch.bfloat16):
    if not isinstance(D, torch.Tensor) or not D.is_cuda or not D.is_contiguous() or D.dtype != dtype:
        raise RuntimeError(f"D must be a contiguous CUDA {dtype} tensor")
    if tuple(D.shape) != (M, N):
        raise RuntimeError(f"D must have shape ({M}, {N}), got {tuple(D.shape)}")


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


class _NoPdl:
    """The GEMM launches inside the block are ordinary launches, not programmatic dependents (the reference's
    ``*_nopdl`` entry points, nvfp4_b200_gemm.cu:1702-1735); the calling thread's setting is restored afterwards."""

    def __enter__(self):
        self._before = _lib.load().fp4b200_set_gemm_pdl(0)

    def __exit__(self, *exc):
        _lib.load().fp4b200_set_gemm_pdl(self._before)
        return False


def _gemm(A, A_sc, A_sg, B, B_sc, B_sg, D, residual=None):
    for t, n in ((A, "A"), (A_sc, "A_sc"), (B, "B"), (B_sc, "B_sc")):
        _chk_operand(t, n)
    _chk_sg(A_sg, "A_sc_global")
    _chk_sg(B_sg, "B_sc_global")
    M, N, K = _shapes(A, B)
    out_fp32 = 1 if D.dtype == torch.float32 else 0
    _chk_out(D, M, N, D.dtype if out_fp32 else torch.bfloat16)
    if residual is not None:
        _chk_out(residual, M, N)
    with torch.cuda.device(A.device):
        _lib.call("fp4b200_nvfp4_gemm", A.data_ptr(), A_sc.data_ptr(), A_sg.data_ptr(), B.data_ptr(),
                  B_sc.data_ptr(), B_sg.data_ptr(), D.data_ptr(), out_fp32,
                  None if residual is None else residual.data_ptr(), M, N, K, _stream(A))


def nvfp4_gemm(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D):
    """nvfp4_b200_gemm.cu:648-761.  A float32 ``D`` selects the unrounded fp32 epilogue (an
    addition used by the parity tests; the reference writes bf16 only)."""
    _gemm(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D)


def nvfp4_gemm_config(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D, config_id):
    """nvfp4_b200_gemm.cu:1899-1920.  ``config_id`` selects among the reference's precompiled tile
    shapes; this library has one tile shape, so the id is accepted and ignored."""
    _gemm(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D)


def nvfp4_gemm_nopdl(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D):
    with _NoPdl():
        _gemm(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D)


def nvfp4_gemm_config_nopdl(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D, config_id):
    with _NoPdl():
        _gemm(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D)


def nvfp4_gemm_residual(A, A_sc, A_sc_global, B, B_sc, B_sc_global, R, D):
    """nvfp4_b200_gemm.cu:1702-1735: ``D = bf16(bf16(acc * sg) + R)``."""
    _gemm(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D, residual=R)


def nvfp4_grouped_gemm(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, D, D_K_opt=None, D_V_opt=None, silu_dim=0):
    """nvfp4_b200_gemm.cu:764-841: one GEMM over concatenated weights, per-256-row tensor scales,
    outputs routed by column range to ``D`` (and ``D_K_opt``, ``D_V_opt``); ``silu_dim`` > 0 applies
    ``x / (1 + exp(-x))`` to the first ``silu_dim`` output columns."""
    if silu_dim:
        # SiLU of the columns [0, silu_dim) in the epilogue (nvfp4_gemm.cuh:210-225)
        outs = [D] + [t for t in (D_K_opt, D_V_opt) if t is not None]
        return _grouped_gemm_rope(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, outs, None, 1, 2, 0, False, silu_dim)
    for t, n in ((A, "A"), (A_sc, "A_sc"), (B, "B"), (B_sc, "B_sc")):
        _chk_operand(t, n)
    M, N, K = _shapes(A, B)
    _chk_sg(A_sc_global, "A_sc_global")
    _chk_sg(B_sg_per_tile, "B_sg_per_tile", N // 256)
    outs = [D] + [t for t in (D_K_opt, D_V_opt) if t is not None]
    cols = []
    for o in outs:
        if not o.is_cuda or o.dtype != torch.bfloat16 or not o.is_contiguous() or o.dim() != 2 or o.shape[0] != M:
            raise RuntimeError("grouped GEMM outputs must be contiguous CUDA bfloat16 [M, n_i]")
        cols.append(o.shape[1])
    if sum(cols) != N:
        raise RuntimeError(f"grouped GEMM outputs have {sum(cols)} columns in total, B has {N} rows")
    ptrs = (ctypes.c_void_p * len(outs))(*[o.data_ptr() for o in outs])
    ccols = (ctypes.c_int64 * len(outs))(*cols)
    with torch.cuda.device(A.device):
        _lib.call("fp4b200_nvfp4_grouped_gemm", A.data_ptr(), A_sc.data_ptr(), A_sc_global.data_ptr(), B.data_ptr(),
                  B_sc.data_ptr(), B_sg_per_tile.data_ptr(), len(outs), ptrs, ccols, M, N, K, _stream(A))


def nvfp4_grouped_gemm_nopdl(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, D, D_K_opt=None, D_V_opt=None,
                             silu_dim=0):
    with _NoPdl():
        nvfp4_grouped_gemm(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, D, D_K_opt, D_V_opt, silu_dim)


def nvfp4_grouped_gemm_config_nopdl(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, D, D_K_opt=None, D_V_opt=None,
                                    silu_dim=0, config_id=5):
    """nvfp4_b200_gemm.cu:2922-2927 — the non-PDL grouped GEMM with the reference's tile-configuration index, which is
    accepted and ignored (one tile configuration here)."""
    nvfp4_grouped_gemm_nopdl(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, D, D_K_opt, D_V_opt, silu_dim)


def _grouped_gemm_rope(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, outs, rope_cs, seq_len, head_dim, rope_cols,
                       round_input_bf16, silu_dim=0):
    for t, n in ((A, "A"), (A_sc, "A_sc"), (B, "B"), (B_sc, "B_sc")):
        _chk_operand(t, n)
    M, N, K = _shapes(A, B)
    _chk_sg(A_sc_global, "A_sc_global")
    _chk_sg(B_sg_per_tile, "B_sg_per_tile", N // 256)
    cols = []
    for o in outs:
        if not o.is_cuda or o.dtype != torch.bfloat16 or not o.is_contiguous() or o.dim() != 2 or o.shape[0] != M:
            raise RuntimeError("Q/K/V outputs must be contiguous CUDA bfloat16 [M, n_i]")
        cols.append(o.shape[1])
    if sum(cols) != N:
        raise RuntimeError("Q/K/V output columns must sum to B rows")
    seq_len, head_dim = int(seq_len), int(head_dim)
    if rope_cs is not None:
        if seq_len <= 0 or seq_len & (seq_len - 1):
            raise RuntimeError("rope_seq_len must be a power of two")
        if (not rope_cs.is_cuda or not rope_cs.is_contiguous() or rope_cs.dtype != torch.float32
                or tuple(rope_cs.shape) != (seq_len, head_dim // 2, 2)):
            raise RuntimeError("rope_cs must be contiguous CUDA float32 [seq_len,rotary_dim/2,2]")
    ptrs = (ctypes.c_void_p * len(outs))(*[o.data_ptr() for o in outs])
    ccols = (ctypes.c_int64 * len(outs))(*cols)
    with torch.cuda.device(A.device):
        _lib.call("fp4b200_nvfp4_grouped_gemm_rope", A.data_ptr(), A_sc.data_ptr(), A_sc_global.data_ptr(), B.data_ptr(),
                  B_sc.data_ptr(), B_sg_per_tile.data_ptr(), len(outs), ptrs, ccols,
                  None if rope_cs is None else rope_cs.data_ptr(), seq_len, head_dim, int(rope_cols),
                  int(bool(round_input_bf16)), int(silu_dim), M, N, K, _stream(A))


def nvfp4_grouped_gemm_rope_live64(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, D, D_K, D_V, rope_cs, rope_seq_len,
                                   silu_dim=0):
    """nvfp4_b200_gemm.cu:1338-1368 — fused QKV projection, rotary embedding (heads of 64) on the Q and K outputs in
    the epilogue, V untouched; rope_cs [seq_len, 32, 2]."""
    _grouped_gemm_rope(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, [D, D_K, D_V], rope_cs, rope_seq_len, 64,
                       D.shape[1] + D_K.shape[1], False, silu_dim)


def nvfp4_grouped_gemm_rope_packed_split(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, D, D_K, D_V, rope_cs, rope_seq_len,
                                         rope_head_dim, rope_rotary_dim):
    """nvfp4_b200_gemm.cu:1406-1441 — as above for any power-of-two head size, the scaled accumulator rounded to
    bf16 before the rotation (the order of the unfused path: GEMM output in bf16, then RoPE)."""
    if int(rope_rotary_dim) != int(rope_head_dim):
        raise RuntimeError("packed RoPE requires rotary_dim == head_dim")
    _grouped_gemm_rope(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, [D, D_K, D_V], rope_cs, rope_seq_len, rope_head_dim,
                       D.shape[1] + D_K.shape[1], True)


def nvfp4_grouped_gemm_rope_packed_cat(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, D, rope_cs, rope_seq_len,
                                       rope_head_dim, rope_rotary_dim, q_dim, k_dim):
    """nvfp4_b200_gemm.cu:1370-1404 — single output [M, q_dim + k_dim + v_dim], rotation on the first q_dim + k_dim
    columns."""
    if int(rope_rotary_dim) != int(rope_head_dim):
        raise RuntimeError("packed RoPE requires rotary_dim == head_dim")
    q_dim, k_dim = int(q_dim), int(k_dim)
    if q_dim <= 0 or k_dim <= 0 or q_dim + k_dim >= B.shape[0] or q_dim % 256 or k_dim % 256:
        raise RuntimeError("Q/K dimensions must be positive multiples of 256 with a V suffix")
    _grouped_gemm_rope(A, A_sc, A_sc_global, B, B_sc, B_sg_per_tile, [D], rope_cs, rope_seq_len, rope_head_dim,
                       q_dim + k_dim, True)


def _rope_packed_qk(q, k, rope_cs, rope_seq_len, rope_head_dim, q_out, k_out, inverse):
    for t in (q, k, q_out, k_out):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or not t.is_contiguous():
            raise RuntimeError("Q/K inputs and outputs must be contiguous CUDA bf16 matrices")
    if q.shape != q_out.shape or k.shape != k_out.shape:
        raise RuntimeError("Q/K output shapes must match their inputs")
    if q.shape[0] != k.shape[0]:
        raise RuntimeError("Q/K rows must match")
    seq_len, head = int(rope_seq_len), int(rope_head_dim)
    if (not rope_cs.is_cuda or not rope_cs.is_contiguous() or rope_cs.dtype != torch.float32
            or tuple(rope_cs.shape) != (seq_len, head // 2, 2)):
        raise RuntimeError("rope_cs must be contiguous CUDA float32 [seq_len,head_dim/2,2]")
    for out in (q_out, k_out):
        for src in (q, k):
            if out.data_ptr() < src.data_ptr() + src.numel() * 2 and src.data_ptr() < out.data_ptr() + out.numel() * 2:
                raise RuntimeError("output must not overlap an input")
    with torch.cuda.device(q.device):
        _lib.call("fp4b200_rope_packed_qk", q.data_ptr(), k.data_ptr(), rope_cs.data_ptr(), seq_len, head, q_out.data_ptr(),
                  k_out.data_ptr(), q.shape[0], q.shape[1], k.shape[1], int(inverse), _stream(q))


def nvfp4_forward_rope_packed_qk(q, k, rope_cs, rope_seq_len, rope_head_dim, q_out, k_out):
    """nvfp4_b200_gemm.cu:1183-1194 — rotary embedding of contiguous bf16 Q and K in one launch."""
    _rope_packed_qk(q, k, rope_cs, rope_seq_len, rope_head_dim, q_out, k_out, False)


def nvfp4_inverse_rope_packed_qk(q, k, rope_cs, rope_seq_len, rope_head_dim, q_out, k_out):
    """nvfp4_b200_gemm.cu:1205-1216 — the inverse rotation (gradients of Q and K on the way back to the QKV dgrad)."""
    _rope_packed_qk(q, k, rope_cs, rope_seq_len, rope_head_dim, q_out, k_out, True)


def nvfp4_batched_gemm(A_list, A_sc_list, A_sg_list, B_list, B_sc_list, B_sg_list, D_list):
    """nvfp4_b200_gemm.cu:1946-2010: independent GEMMs ``D_i = A_i . B_i^T`` (up to four)."""
    n = len(D_list)
    if not (len(A_list) == len(A_sc_list) == len(A_sg_list) == len(B_list) == len(B_sc_list) == len(B_sg_list) == n):
        raise RuntimeError("nvfp4_batched_gemm: all lists must have the same length")
    for i in range(n):
        _gemm(A_list[i], A_sc_list[i], A_sg_list[i], B_list[i], B_sc_list[i], B_sg_list[i], D_list[i])


def nvfp4_batched_accum_gemm(A_list, A_sc_list, A_sg_list, B_list, B_sc_list, B_sg_list, D_out):
    """nvfp4_b200_gemm.cu:2567-2635: ``D_out = bf16(sum_i (A_i . B_i^T) * A_sg_i * B_sg_i)`` with the sum kept in
    fp32 in batch order — term 0 multiplied, every later term joined by one fused multiply-add, as the reference's
    kernel does.  Up to four terms with M a multiple of 256 run as ONE launch (the terms' accumulators are summed in
    the epilogue's registers); anything else as a chain of launches through an fp32 partial sum."""
    n = len(A_list)
    if n == 0 or not (len(A_sc_list) == len(A_sg_list) == len(B_list) == len(B_sc_list) == len(B_sg_list) == n):
        raise RuntimeError("nvfp4_batched_accum_gemm: all lists must have the same non-zero length")
    if n == 1:
        return _gemm(A_list[0], A_sc_list[0], A_sg_list[0], B_list[0], B_sc_list[0], B_sg_list[0], D_out)
    M, N, _ = _shapes(A_list[0], B_list[0])
    _chk_out(D_out, M, N)
    Ks = []
    for i in range(n):
        for t, nm in ((A_list[i], "A"), (A_sc_list[i], "A_sc"), (B_list[i], "B"), (B_sc_list[i], "B_sc")):
            _chk_operand(t, nm)
        _chk_sg(A_sg_list[i], "A_sc_global")
        _chk_sg(B_sg_list[i], "B_sc_global")
        Mi, Ni, Ki = _shapes(A_list[i], B_list[i])
        if (Mi, Ni) != (M, N):
            raise RuntimeError("nvfp4_batched_accum_gemm: every term must produce the same [M, N]")
        Ks.append(Ki)
    with torch.cuda.device(D_out.device):
        if n <= 4 and M % 256 == 0 and os.environ.get("FP4B200_GEMM_PAIR", "1") != "0":
            def arr(ts):
                return (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
            _lib.call("fp4b200_nvfp4_batched_accum_gemm", n, arr(A_list), arr(A_sc_list), arr(A_sg_list), arr(B_list),
                      arr(B_sc_list), arr(B_sg_list), (ctypes.c_int64 * n)(*Ks), None, None, D_out.data_ptr(), M, N, 0,
                      _stream(A_list[0]))
            return
        partial = torch.empty((M, N), dtype=torch.float32, device=D_out.device)
        _gemm(A_list[0], A_sc_list[0], A_sg_list[0], B_list[0], B_sc_list[0], B_sg_list[0], partial)
        for i in range(1, n):
            last = i == n - 1
            dst = D_out if last else partial
            _lib.call("fp4b200_nvfp4_gemm_accum", A_list[i].data_ptr(), A_sc_list[i].data_ptr(), A_sg_list[i].data_ptr(),
                      B_list[i].data_ptr(), B_sc_list[i].data_ptr(), B_sg_list[i].data_ptr(), partial.data_ptr(),
                      dst.data_ptr(), 0 if last else 1, M, N, Ks[i], _stream(A_list[i]))


def nvfp4_split_dgrad_sum(A_fp4_cat, A_sc_cat, A_sg_list, B_fp4_list, B_sc_list, B_sg_cat, split_dims, D_out):
    """nvfp4_b200_gemm.cu:2424-2565: dgrad of a fused projection — the row-quantised gradient is the column
    concatenation of the splits; term i multiplies columns of split i by the column-quantised weight i.  The
    reference multiplies every split into a bf16 matrix of its own and adds those with ``Tensor.add_``, so every term
    and every partial sum is rounded to bf16; so here.  One launch over the column slices where they are (M a multiple
    of 256, up to four splits; the epilogue rounds as described); otherwise one GEMM per split and ``add_``."""
    n = len(split_dims)
    if any(d % 128 for d in split_dims):
        raise RuntimeError("nvfp4_split_dgrad_sum: split sizes must be multiples of 128")
    a_u8 = A_fp4_cat.view(torch.uint8)
    sc_u8 = A_sc_cat.view(torch.uint8)
    M, k_total = a_u8.shape[0], a_u8.shape[1] * 2
    one_launch = (n <= 4 and M % 256 == 0 and os.environ.get("FP4B200_GEMM_PAIR", "1") != "0" and a_u8.is_contiguous()
                  and sc_u8.is_contiguous() and all(d % 256 == 0 for d in split_dims)
                  and sum(split_dims) == k_total and len(B_fp4_list) == n and len(B_sc_list) == n and len(A_sg_list) == n)
    if one_launch:
        N = B_fp4_list[0].shape[0]
        _chk_out(D_out, M, N)
        for i in range(n):
            for t, nm in ((B_fp4_list[i], "B"), (B_sc_list[i], "B_sc")):
                _chk_operand(t, nm)
            _chk_sg(A_sg_list[i], "A_sc_global")
            if B_fp4_list[i].shape != (N, split_dims[i] // 2):
                raise RuntimeError("nvfp4_split_dgrad_sum: weight i must be [N, split_i / 2] codes")
        _chk_sg(B_sg_cat, "B_sg_cat", n)
        offs, a_ptrs, sc_ptrs = 0, [], []
        for d in split_dims:
            a_ptrs.append(a_u8.data_ptr() + offs // 2)
            sc_ptrs.append(sc_u8.data_ptr() + (offs // 64) * 512)
            offs += d
        vp = ctypes.c_void_p * n
        i64 = ctypes.c_int64 * n
        with torch.cuda.device(D_out.device):
            _lib.call("fp4b200_nvfp4_batched_accum_gemm", n, vp(*a_ptrs), vp(*sc_ptrs), vp(*[t.data_ptr() for t in A_sg_list]),
                      vp(*[t.data_ptr() for t in B_fp4_list]), vp(*[t.data_ptr() for t in B_sc_list]),
                      vp(*[B_sg_cat.data_ptr() + 4 * i for i in range(n)]), i64(*split_dims), i64(*([k_total // 2] * n)),
                      i64(*([k_total // 64] * n)), D_out.data_ptr(), M, N, 1, _stream(A_fp4_cat))
        return
    # as the reference: one GEMM per split into a bf16 matrix of its own, then Tensor.add_ left to right
    offs = 0
    for i, d in enumerate(split_dims):
        a_i = a_u8[:, offs // 2:(offs + d) // 2].contiguous()
        sc_i = sc_u8[:, offs // 64:(offs + d) // 64, :].contiguous()
        if i == 0:
            _gemm(a_i, sc_i, A_sg_list[i], B_fp4_list[i], B_sc_list[i], B_sg_cat.narrow(0, i, 1), D_out)
        else:
            term = torch.empty_like(D_out)
            _gemm(a_i, sc_i, A_sg_list[i], B_fp4_list[i], B_sc_list[i], B_sg_cat.narrow(0, i, 1), term)
            D_out.add_(term)
        offs += d


def nvfp4_row_rms_reduce(row_rms_partial, coeff, hidden_size, eps):
    """nvfp4_b200_gemm.cu:1792-1803 — coeff[r] = rsqrt(sum(row_rms_partial[r, :]) / hidden_size + eps), in place."""
    if (not isinstance(coeff, torch.Tensor) or not coeff.is_cuda or coeff.dtype != torch.float32 or coeff.dim() != 1
            or not coeff.is_contiguous() or coeff.shape[0] != row_rms_partial.shape[0]):
        raise RuntimeError("coeff must be contiguous CUDA float32 [M]")
    p = row_rms_partial
    if not p.is_cuda or p.dtype != torch.float32 or p.dim() != 2 or not p.is_contiguous() or p.device != coeff.device:
        raise RuntimeError("row_rms_partial must be contiguous CUDA float32 [M,P] on coeff's device")
    with torch.cuda.device(p.device):
        _lib.call("fp4b200_row_rms_reduce", p.data_ptr(), p.shape[0], p.shape[1], int(hidden_size), float(eps),
                  coeff.data_ptr(), _stream(p))


def _bf16_matrix(t, name, like=None):
    if (not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous() or t.dtype != torch.bfloat16 or t.dim() != 2
            or (like is not None and (t.shape != like.shape or t.device != like.device))):
        raise RuntimeError(f"{name} must be contiguous CUDA bf16 [M,K]")


def sum3_rmsnorm_bwd_out(d0, d1, d2, input, norm_weight, inv_rms, d_sum, grad_input, dgamma_partials, dgamma):
    """nvfp4_b200_gemm.cu:432-562 — d_sum = d0 + d1 + d2 (bf16, left to right), RMSNorm backward dx into grad_input,
    dgamma through fixed 256-row tiles (dgamma_partials [ceil(M/256), K] fp32) into dgamma [K] (fp32 or bf16);
    everything into the caller's tensors."""
    _bf16_matrix(d0, "d0")
    for t, name in ((d1, "d1"), (d2, "d2"), (input, "input"), (d_sum, "d_sum"), (grad_input, "grad_input")):
        _bf16_matrix(t, name, d0)
    M, K = d0.shape
    if M <= 0 or K <= 0:
        raise RuntimeError("sum3_rmsnorm_bwd_out requires positive int32-indexable M*K")
    if (not norm_weight.is_cuda or not norm_weight.is_contiguous() or norm_weight.dtype != torch.bfloat16
            or norm_weight.dim() != 1 or norm_weight.numel() != K):
        raise RuntimeError("norm_weight must be contiguous CUDA bf16 [K]")
    if not inv_rms.is_cuda or not inv_rms.is_contiguous() or inv_rms.dtype != torch.float32 or inv_rms.numel() != M:
        raise RuntimeError("inv_rms must be contiguous CUDA fp32 [M]")
    tiles = (M + 255) // 256
    if (not dgamma_partials.is_cuda or not dgamma_partials.is_contiguous() or dgamma_partials.dtype != torch.float32
            or tuple(dgamma_partials.shape) != (tiles, K)):
        raise RuntimeError("dgamma_partials must be contiguous CUDA fp32 [ceil(M/256),K]")
    if (not dgamma.is_cuda or not dgamma.is_contiguous() or dgamma.dtype not in (torch.float32, torch.bfloat16)
            or dgamma.dim() != 1 or dgamma.numel() != K):
        raise RuntimeError("dgamma must be contiguous CUDA fp32 or bf16 [K]")
    with torch.cuda.device(d0.device):
        _lib.call("fp4b200_sum3_rmsnorm_bwd", d0.data_ptr(), d1.data_ptr(), d2.data_ptr(), input.data_ptr(),
                  norm_weight.data_ptr(), inv_rms.data_ptr(), d_sum.data_ptr(), grad_input.data_ptr(),
                  dgamma_partials.data_ptr(), dgamma.data_ptr(), int(dgamma.dtype == torch.bfloat16), M, K, _stream(d0))


def rmsnorm_bwd_residual_out(d_normed, input, norm_weight, inv_rms, residual_grad, grad_input, dgamma):
    """nvfp4_b200_gemm.cu:564-646 — grad_input = bf16(RMSNorm backward dx) + residual_grad, dgamma [4096] fp32; K = 4096.
    dgamma is accumulated through fixed 256-row tiles (a scratch tensor from torch's allocator) instead of the
    reference's atomics, so repeated calls give identical bits."""
    _bf16_matrix(d_normed, "d_normed")
    M, K = d_normed.shape
    if M <= 0 or K != 4096:
        raise RuntimeError("rmsnorm_bwd_residual_out requires [M,4096] with int32 M")
    for t, name in ((input, "input"), (residual_grad, "residual_grad"), (grad_input, "grad_input")):
        _bf16_matrix(t, name, d_normed)
    if (not norm_weight.is_cuda or not norm_weight.is_contiguous() or norm_weight.dtype != torch.bfloat16
            or norm_weight.dim() != 1 or norm_weight.numel() != K):
        raise RuntimeError("norm_weight must be contiguous CUDA bf16 [4096]")
    if (not inv_rms.is_cuda or not inv_rms.is_contiguous() or inv_rms.dtype != torch.float32 or inv_rms.dim() != 1
            or inv_rms.numel() != M):
        raise RuntimeError("inv_rms must be contiguous CUDA fp32 [M]")
    if not dgamma.is_cuda or not dgamma.is_contiguous() or dgamma.dtype != torch.float32 or dgamma.dim() != 1 or dgamma.numel() != K:
        raise RuntimeError("dgamma must be contiguous CUDA fp32 [4096]")
    partials = torch.empty(((M + 255) // 256, K), dtype=torch.float32, device=d_normed.device)
    with torch.cuda.device(d_normed.device):
        _lib.call("fp4b200_rmsnorm_bwd_residual", d_normed.data_ptr(), input.data_ptr(), norm_weight.data_ptr(),
                  inv_rms.data_ptr(), residual_grad.data_ptr(), grad_input.data_ptr(), partials.data_ptr(), dgamma.data_ptr(),
                  M, K, _stream(d_normed))


def fp32_to_fp4x2(A_fp32):
    """nvfp4_b200_gemm.cu:1480-1494 — [R, C] float32 -> [R, C/2] float4_e2m1fn_x2 (RN-even, saturating)."""
    if not A_fp32.is_cuda or A_fp32.dtype != torch.float32 or A_fp32.dim() != 2 or not A_fp32.is_contiguous() \
            or A_fp32.shape[1] % 2:
        raise RuntimeError("fp32_to_fp4x2 expects a contiguous CUDA float32 [R, C] with even C")
    out = torch.empty((A_fp32.shape[0], A_fp32.shape[1] // 2), dtype=torch.uint8, device=A_fp32.device)
    with torch.cuda.device(A_fp32.device):
        _lib.call("fp4b200_fp32_to_fp4x2", A_fp32.data_ptr(), out.numel(), out.data_ptr(), _stream(A_fp32))
    return out.view(torch.float4_e2m1fn_x2)


def fp4x2_to_fp32(A_fp4x2):
    """nvfp4_b200_gemm.cu:1496-1510 — [R, C/2] packed codes -> [R, C] float32."""
    a = A_fp4x2.view(torch.uint8)
    if not a.is_cuda or a.dim() != 2 or not a.is_contiguous():
        raise RuntimeError("fp4x2_to_fp32 expects a contiguous CUDA [R, C/2] tensor of packed codes")
    out = torch.empty((a.shape[0], a.shape[1] * 2), dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        _lib.call("fp4b200_fp4x2_to_fp32", a.data_ptr(), a.numel(), out.data_ptr(), _stream(a))
    return out


def nvfp4_quantize(A_bf16, A_fp4x2, A_sc, A_sc_global, scale_2d):
    """nvfp4_b200_gemm.cu:1443-1478 — the GEMM module's own operand producer (used by its tests): fills the
    caller's A_fp4x2 [M, N/2], A_sc (512-byte scale tiles, [M/128, N/64, 512] bytes) and A_sc_global [1]."""
    if not A_bf16.is_cuda or A_bf16.dtype != torch.bfloat16 or A_bf16.dim() != 2 or not A_bf16.is_contiguous():
        raise RuntimeError("A_bf16 must be a contiguous CUDA bfloat16 [M, N]")
    M, N = A_bf16.shape
    fp4 = A_fp4x2.view(torch.uint8)
    sc = A_sc.view(torch.uint8)
    if tuple(fp4.shape) != (M, N // 2) or not fp4.is_contiguous() or sc.numel() != M * N // 16 or not sc.is_contiguous():
        raise RuntimeError("A_fp4x2 must be [M, N/2] and A_sc must hold M*N/16 scale bytes, both contiguous")
    if A_sc_global.dtype != torch.float32 or A_sc_global.numel() != 1:
        raise RuntimeError("A_sc_global must be a float32 tensor with one element")
    with torch.cuda.device(A_bf16.device):
        _lib.call("fp4b200_tk_nvfp4_quantize", A_bf16.data_ptr(), M, N, fp4.data_ptr(), sc.data_ptr(),
                  A_sc_global.data_ptr(), int(bool(scale_2d)), _stream(A_bf16))

