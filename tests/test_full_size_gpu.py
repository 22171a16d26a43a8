"""Full-size runs at the benchmark configurations (M = 16384 tokens, K = 4096, H = 14336), checked
through properties that do not need a full-size CPU reference: sampled rows x columns of every GEMM
against the oracle's product of the same quantised bytes (relative Frobenius <= 1e-3 on the sample),
samples from every kind of tile position (first / last / interior row and column tiles), exact
linearity in the tensor scale, determinism, and sampled row blocks of the SwiGLU producer bit-exact
against the oracle."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, u8

pytestmark = pytest.mark.gpu

M_TOK, K_HID, H_FFN = 16384, 4096, 14336


def _randn_bf16(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _sample_indices(n, tile, count, seed):
    """`count` indices out of n covering the first, the last and random interior tiles of size `tile`."""
    rng = np.random.default_rng(seed)
    idx = {0, tile - 1, tile, n - tile, n - 1, n // 2, n // 2 + tile - 1}
    while len(idx) < count:
        idx.add(int(rng.integers(0, n)))
    return np.array(sorted(idx))


def _rows(q_fp4, q_sc, rows, n_rows, K, block=16):
    """Codes and logical scales of the sampled rows of a quantised operand."""
    fp4 = q_fp4.view(torch.uint8)[torch.from_numpy(rows).cuda()].cpu().numpy()
    sc = o.unswizzle_scales(u8(q_sc), n_rows, K // block)[rows]
    return fp4, sc


def _check_sample(d, ref, rows, cols, tol=1e-3):
    got = d[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].float().cpu().numpy()
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= tol, rel
    return rel


def test_config3_gate_up_and_down_gemms_sampled():
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    x = _randn_bf16((M_TOK, K_HID), 1)
    w13 = _randn_bf16((2 * H_FFN, K_HID), 2, 0.02)
    qx = tkq.tk_quantize_for_gemm(x, False, True)
    q1 = tkq.tk_quantize_for_gemm(w13[:H_FFN].contiguous(), False, True)
    q3 = tkq.tk_quantize_for_gemm(w13[H_FFN:].contiguous(), False, True)
    b = torch.cat([q1[0].view(torch.uint8), q3[0].view(torch.uint8)], 0)
    b_sc = torch.cat([q1[1].view(torch.uint8), q3[1].view(torch.uint8)], 0)
    b_sg = torch.cat([q1[4].expand(H_FFN // 256), q3[4].expand(H_FFN // 256)]).contiguous()
    h1 = torch.empty((M_TOK, H_FFN), dtype=torch.bfloat16, device="cuda")
    h3 = torch.empty((M_TOK, H_FFN), dtype=torch.bfloat16, device="cuda")
    gemm.nvfp4_grouped_gemm(qx[0], qx[1], qx[4], b, b_sc, b_sg, h1, h3)
    f1 = torch.empty((M_TOK, H_FFN), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], q1[0], q1[1], q1[4], f1)   # fp32 epilogue of the first half
    torch.cuda.synchronize()
    assert_status_ok()
    rows = _sample_indices(M_TOK, 256, 48, 11)
    cols = _sample_indices(H_FFN, 256, 64, 12)
    a_fp4, a_sc = _rows(qx[0], qx[1], rows, M_TOK, K_HID)
    for q, d in ((q1, h1), (q3, h3)):
        w_fp4, w_sc = _rows(q[0], q[1], cols, H_FFN, K_HID)
        ref = o.nvfp4_gemm_fp32(a_fp4, a_sc, qx[4].item(), w_fp4, w_sc, q[4].item())
        _check_sample(d, o.bf16_round(ref), rows, cols, tol=3e-3)   # bf16 output: one rounding on top of the fp32 result
        if q is q1:
            assert _check_sample(f1, ref, rows, cols) < 1e-5
    # the grouped launch equals the plain one, rounded
    assert torch.equal(h1, f1.to(torch.bfloat16))
    # linearity in the tensor scale: doubling A_sg doubles the fp32 output exactly
    f1b = torch.empty_like(f1)
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4] * 2, q1[0], q1[1], q1[4], f1b)
    torch.cuda.synchronize()
    assert torch.equal(f1b, f1 * 2)
    del f1b, f1, h3

    # down projection: K = 14336 (bf16 output as in the forward pass)
    h = _randn_bf16((M_TOK, H_FFN), 3)
    w2 = _randn_bf16((K_HID, H_FFN), 4, 0.02)
    qh = tkq.tk_quantize_for_gemm(h, False, True)
    q2 = tkq.tk_quantize_for_gemm(w2, False, True)
    y = torch.empty((M_TOK, K_HID), dtype=torch.bfloat16, device="cuda")
    gemm.nvfp4_gemm(qh[0], qh[1], qh[4], q2[0], q2[1], q2[4], y)
    y2 = torch.empty_like(y)
    gemm.nvfp4_gemm(qh[0], qh[1], qh[4], q2[0], q2[1], q2[4], y2)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    cols2 = _sample_indices(K_HID, 256, 64, 13)
    a_fp4, a_sc = _rows(qh[0], qh[1], rows, M_TOK, H_FFN)
    w_fp4, w_sc = _rows(q2[0], q2[1], cols2, K_HID, H_FFN)
    ref = o.nvfp4_gemm_fp32(a_fp4, a_sc, qh[4].item(), w_fp4, w_sc, q2[4].item())
    _check_sample(y, o.bf16_round(ref), rows, cols2, tol=3e-3)   # bf16 output: one rounding on top of the fp32 result
    assert_status_ok()


def test_config4_wgrad_gemm_from_column_operands_sampled():
    """dW2 [K_HID, H_FFN] = dY^T . h: both operands are the column-wise (transposed) quantisations, the
    contraction runs over the 16384 tokens."""
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    dy = _randn_bf16((M_TOK, K_HID), 5, 1e-3)
    h = _randn_bf16((M_TOK, H_FFN), 6)
    qd = tkq.tk_quantize_for_gemm(dy, True, False)
    qh = tkq.tk_quantize_for_gemm(h, True, False)
    dw = torch.empty((K_HID, H_FFN), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qd[2], qd[3], qd[4], qh[2], qh[3], qh[4], dw)
    torch.cuda.synchronize()
    assert_status_ok()
    rows = _sample_indices(K_HID, 256, 48, 21)
    cols = _sample_indices(H_FFN, 256, 64, 22)
    a_fp4, a_sc = _rows(qd[2], qd[3], rows, K_HID, M_TOK)
    b_fp4, b_sc = _rows(qh[2], qh[3], cols, H_FFN, M_TOK)
    ref = o.nvfp4_gemm_fp32(a_fp4, a_sc, qd[4].item(), b_fp4, b_sc, qh[4].item())
    assert _check_sample(dw, ref, rows, cols) < 1e-5


def test_config3_swiglu_producer_sampled_blocks():
    tkq = mod("tk_quant_v5")
    h1 = _randn_bf16((M_TOK, H_FFN), 7, 2.0)
    h3 = _randn_bf16((M_TOK, H_FFN), 8)
    out = tkq.tk_silu_quantize_split_for_gemm(h1, h3)
    h = out[8]
    out2 = tkq.tk_silu_quantize_split_for_gemm(h1, h3)
    torch.cuda.synchronize()
    assert_status_ok()
    for i in range(4):
        assert torch.equal(out[i].view(torch.uint8), out2[i].view(torch.uint8))   # determinism
    amax = out[6][0].item()
    assert amax == h.float().abs().max().item() and out[4].item() == np.float32(amax) / np.float32(2688.0)
    # the quantiser's bytes for sampled 128-row blocks, from the materialised h and the tensor amax
    row_sc = u8(out[1]).reshape(M_TOK // 128, H_FFN // 64, 512)
    for blk in (0, 37, M_TOK // 128 - 1):
        hb = h[blk * 128:(blk + 1) * 128].float().cpu().numpy()
        fp4, sc = o.nvfp4_quantize_1d(hb, amax, "encode")
        assert np.array_equal(u8(out[0][blk * 128:(blk + 1) * 128]), fp4)
        assert np.array_equal(row_sc[blk], o.swizzle_scales(sc)[0])
    # column operand: sampled 128-column blocks against the transposed slice
    col_sc = u8(out[3]).reshape(H_FFN // 128, M_TOK // 64, 512)
    for blk in (0, 55, H_FFN // 128 - 1):
        ht = np.ascontiguousarray(h[:, blk * 128:(blk + 1) * 128].float().cpu().numpy().T)
        fp4, sc = o.nvfp4_quantize_1d(ht, amax, "encode")
        assert np.array_equal(u8(out[2][blk * 128:(blk + 1) * 128]), fp4)
        assert np.array_equal(col_sc[blk], o.swizzle_scales(sc)[0])


def test_config5_mxfp4_gemm_sampled():
    """One rank's slice of the MXFP4 layer set: M = 8192 tokens, W1 [14336, 4096], mode 1."""
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    M = 8192
    x = _randn_bf16((M, K_HID), 9)
    w = _randn_bf16((H_FFN, K_HID), 10, 0.02)
    qx = mxq.mxfp4_quantize_for_gemm(x, 1)
    qw = mxq.mxfp4_quantize_for_gemm(w, 1)
    d = torch.empty((M, H_FFN), dtype=torch.float32, device="cuda")
    gemm.mxfp4_gemm(qx[0], qx[1], qw[0], qw[1], d)
    torch.cuda.synchronize()
    assert_status_ok()
    rows = _sample_indices(M, 256, 48, 31)
    cols = _sample_indices(H_FFN, 256, 64, 32)
    a_fp4, a_e = _rows(qx[0], qx[1].reshape(M // 128, K_HID // 128, 512), rows, M, K_HID, block=32)
    b_fp4, b_e = _rows(qw[0], qw[1].reshape(H_FFN // 128, K_HID // 128, 512), cols, H_FFN, K_HID, block=32)
    ref = o.mxfp4_gemm_fp32(a_fp4, a_e, b_fp4, b_e)
    assert _check_sample(d, ref, rows, cols) < 1e-5
