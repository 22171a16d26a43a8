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


def mxfp4_gemm_rope_live64(A, A_sc, B, B_sc, D, rope_cs, rope_seq_len):
    """mxfp4_gb200_gemm.cu:1777-1787 — ``D = bf16(rope((A . B^T) / 36))``: every neighbouring column pair of the output
    rotated in fp32 before the one rounding; ``rope_cs`` fp32 [rope_seq_len, head_dim/2, 2], the head size (a power
    of two) read off its shape."""
    for t, n in ((A, "A"), (A_sc, "A_sc"), (B, "B"), (B_sc, "B_sc")):
        _chk_operand(t, n)
    M, N, K = _shapes(A, B)
    _chk_out(D, M, N)
    seq = int(rope_seq_len)
    if seq <= 0 or seq & (seq - 1):
        raise RuntimeError("rope_seq_len must be a power of two")
    if M % seq:
        raise RuntimeError("output rows must be divisible by rope_seq_len")
    if (not isinstance(rope_cs, torch.Tensor) or not rope_cs.is_cuda or not rope_cs.is_contiguous()
            or rope_cs.dtype != torch.float32 or rope_cs.dim() != 3 or rope_cs.shape[0] != seq or rope_cs.shape[2] != 2):
        raise RuntimeError("rope_cs must be contiguous CUDA float32 [rope_seq_len, head_dim/2, 2]")
    head = 2 * int(rope_cs.shape[1])
    if head & (head - 1) or N % head:
        raise RuntimeError("output cols must be divisible by the RoPE head dimension")
    with torch.cuda.device(A.device):
        _lib.call("fp4b200_mxfp4_gemm_rope", A.data_ptr(), A_sc.data_ptr(), B.data_ptr(), B_sc.data_ptr(), D.data_ptr(),
                  rope_cs.data_ptr(), seq, head, M, N, K, _stream(A))


def mxfp4_gemm_rope(A, A_sc, B, B_sc, D, rope_cos, rope_sin, rope_seq_len, rope_head_dim, rope_rotary_dim):
    """mxfp4_gb200_gemm.cu:1814-1827 — the rotary epilogue with separate fp32 tables ``rope_cos`` / ``rope_sin``
    [rope_seq_len, rope_rotary_dim/2].  Built for the full rotation (rotary_dim == head_dim) with power-of-two sequence
    length and head size: the two tables are interleaved into the (cos, sin) table of ``mxfp4_gemm_rope_live64`` (one
    small copy per call); a partial rotary dimension raises."""
    seq, head, rot = int(rope_seq_len), int(rope_head_dim), int(rope_rotary_dim)
    if rot != head:
        raise RuntimeError("mxfp4_gemm_rope: a rotary dimension smaller than the head size is not built")
    if head <= 0 or head & (head - 1) or seq <= 0 or seq & (seq - 1):
        raise RuntimeError("mxfp4_gemm_rope: rope_seq_len and rope_head_dim must be powers of two")
    for t, n in ((rope_cos, "rope_cos"), (rope_sin, "rope_sin")):
        if (not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous() or t.dtype != torch.float32
                or t.numel() != seq * (rot // 2)):
            raise RuntimeError(f"{n} must be contiguous CUDA float32 with rope_seq_len * rope_rotary_dim / 2 elements")
    cs = torch.stack([rope_cos.reshape(seq, rot // 2), rope_sin.reshape(seq, rot // 2)], dim=-1).contiguous()
    mxfp4_gemm_rope_live64(A, A_sc, B, B_sc, D, cs, seq)


def mxfp4_gemm_rope_config(A, A_sc, B, B_sc, D, rope_cos, rope_sin, rope_seq_len, rope_head_dim, rope_rotary_dim, config_id):
    """mxfp4_gb200_gemm.cu:1829-1855 — the same; the tile-configuration index is accepted and ignored."""
    mxfp4_gemm_rope(A, A_sc, B, B_sc, D, rope_cos, rope_sin, rope_seq_len, rope_head_dim, rope_rotary_dim)


def mxfp4_gemm_rope_live64_config(A, A_sc, B, B_sc, D, rope_cs, rope_seq_len, config_id):
    """mxfp4_gb200_gemm.cu:1789-1812 — the same; the tile-configuration index is accepted and ignored."""
    mxfp4_gemm_rope_live64(A, A_sc, B, B_sc, D, rope_cs, rope_seq_len)


mxfp4_gemm_rope_live = mxfp4_gemm_rope_live64                  # mxfp4_gb200_gemm.cu:2824: the same entry point
mxfp4_gemm_rope_live_config = mxfp4_gemm_rope_live64_config    # :2831


def mxfp4_batched_gemm_rope_live64(A_list, A_sc_list, B_list, B_sc_list, D_out_list, rope_cs_list, rope_seq_len_list):
    """mxfp4_gb200_gemm.cu:2958-2964 — independent GEMMs ``D_i = A_i . B_i^T``, each with the rotary epilogue of its own
    table, or plain where its table is empty (the fused QKV projection: Q and K rotated, V not;
    mxfp4_backend.py:3153-3175).  One launch per entry here."""
    for A, A_sc, B, B_sc, D, cs, seq in zip(A_list, A_sc_list, B_list, B_sc_list, D_out_list, rope_cs_list,
                                            rope_seq_len_list, strict=True):
        if cs is None or cs.numel() == 0:
            _gemm(A, A_sc, B, B_sc, D)
        else:
            mxfp4_gemm_rope_live64(A, A_sc, B, B_sc, D, cs, seq)


def mxfp4_batched_gemm_rope_live64_config(A_list, A_sc_list, B_list, B_sc_list, D_out_list, rope_cs_list, rope_seq_len_list,
                                          config_id):
    """mxfp4_gb200_gemm.cu:2965-2972 — the same; the tile-configuration index is accepted and ignored."""
    mxfp4_batched_gemm_rope_live64(A_list, A_sc_list, B_list, B_sc_list, D_out_list, rope_cs_list, rope_seq_len_list)


mxfp4_batched_gemm_rope_live = mxfp4_batched_gemm_rope_live64                  # mxfp4_gb200_gemm.cu:2973
mxfp4_batched_gemm_rope_live_config = mxfp4_batched_gemm_rope_live64_config    # :2980


def mxfp4_gemm_residual_config(A, A_sc, B, B_sc, R, D, config_id):
    """mxfp4_gb200_gemm.cu:2742-2747 — the residual form with the reference's tile-configuration index, which is
    accepted and ignored (one tile configuration here)."""
    _gemm(A, A_sc, B, B_sc, D, residual=R)


def mxfp4_batched_gemm(A_list, A_sc_list, B_list, B_sc_list, D_out_list):
    for A, A_sc, B, B_sc, D in zip(A_list, A_sc_list, B_list, B_sc_list, D_out_list, strict=True):
        _gemm(A, A_sc, B, B_sc, D)


def mxfp4_batched_gemm_config(A_list, A_sc_list, B_list, B_sc_list, D_out_list, config_id):
    mxfp4_batched_gemm(A_list, A_sc_list, B_list, B_sc_list, D_out_list)


def mxfp4_split3_dgrad_strided_onepass_gemm(A_full, A_sc_list, A_col_offsets, A_col_widths, B_list, B_sc_list, D_out,
                                            config_idx=-1):
    """mxfp4_gb200_gemm.cu:2677-2700 — the three-split form (dQ | dK | dV against the three row blocks of the QKV
    weight's column operand): ``D_out = bf16((sum_s A_full[:, off_s:off_s+w_s] . B_s^T) / 36)``, one launch."""
    _split_dgrad_onepass(A_full, A_sc_list, A_col_offsets, A_col_widths, B_list, B_sc_list, D_out, 3)


def mxfp4_split2_dgrad_strided_onepass_gemm(A_full, A_sc_list, A_col_offsets, A_col_widths, B_list, B_sc_list, D_out,
                                            config_idx=-1):
    """mxfp4_gb200_gemm.cu:2572-2596 — ``D_out = bf16((sum_s A_full[:, off_s:off_s+w_s] . B_s^T) / 36)``: the
    row-quantised gradient of a fused projection is the column concatenation of the splits; every term is
    accumulated in tensor memory before the one rounding.  ``A_col_offsets`` / ``A_col_widths`` count PACKED columns
    (bytes of ``A_full``, two elements each), as the reference's do (checks at :430-467).  ``config_idx`` is accepted
    and ignored."""
    _split_dgrad_onepass(A_full, A_sc_list, A_col_offsets, A_col_widths, B_list, B_sc_list, D_out, 2)


def _split_dgrad_onepass(A_full, A_sc_list, A_col_offsets, A_col_widths, B_list, B_sc_list, D_out, want):
    import ctypes
    n = len(B_list)
    if n != want:
        raise RuntimeError(f"split{want} one-pass dgrad expects exactly {want} B tensors")
    if not (len(A_sc_list) == len(A_col_offsets) == len(A_col_widths) == len(B_sc_list) == n):
        raise RuntimeError(f"split{want} one-pass dgrad: list lengths differ")
    _chk_operand(A_full, "A_full")
    for t in list(B_list) + list(B_sc_list):
        _chk_operand(t, "operand")
    # a segment's scales may be a column slice (narrow(1, ...)) of the combined producer's [M/128, tiles, 32, 16] tensor
    row_tiles = []
    for t in A_sc_list:
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError("A_sc_list must hold CUDA tensors")
        if t.is_contiguous():
            row_tiles.append(0)
        elif t.dim() == 4 and tuple(t.shape[2:]) == (32, 16) and tuple(t.stride()[1:]) == (512, 16, 1) and t.stride(0) % 512 == 0:
            row_tiles.append(t.stride(0) // 512)
        else:
            raise RuntimeError("A_sc_list entries must be contiguous or column slices of a [M/128, tiles, 32, 16] tensor")
    a = A_full.view(torch.uint8)
    M, a_width = a.shape[0], a.shape[1] * 2
    N = B_list[0].view(torch.uint8).shape[0]
    for B, w in zip(B_list, A_col_widths):
        b = B.view(torch.uint8)
        if b.shape[0] != N or b.shape[1] != int(w):
            raise RuntimeError("B_list packed K must match A_col_widths")
    for off, w in zip(A_col_offsets, A_col_widths):
        if int(off) < 0 or int(w) <= 0 or int(off) + int(w) > a.shape[1]:
            raise RuntimeError("A_full slice exceeds packed width")
        if (int(w) * 2) % 128:
            raise RuntimeError("split widths must be multiples of 128")
    out_fp32 = 1 if D_out.dtype == torch.float32 else 0
    _chk_out(D_out, M, N, D_out.dtype if out_fp32 else torch.bfloat16)
    offs = (ctypes.c_int64 * n)(*[2 * int(v) for v in A_col_offsets])      # the library counts elements
    widths = (ctypes.c_int64 * n)(*[2 * int(v) for v in A_col_widths])
    a_sc = (ctypes.c_void_p * n)(*[t.data_ptr() for t in A_sc_list])
    b_p = (ctypes.c_void_p * n)(*[t.data_ptr() for t in B_list])
    b_sc = (ctypes.c_void_p * n)(*[t.data_ptr() for t in B_sc_list])
    with torch.cuda.device(A_full.device):
        _lib.call("fp4b200_mxfp4_gemm_ksplit_strided", a.data_ptr(), a_width, n, offs, widths, a_sc,
                  (ctypes.c_int64 * n)(*row_tiles), b_p, b_sc, D_out.data_ptr(), out_fp32, M, N, _stream(A_full))
