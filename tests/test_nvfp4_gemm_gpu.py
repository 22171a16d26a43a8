"""GPU parity: block-scaled FP4 GEMMs through the reference-shaped ``_C`` shim against the oracle's
high-precision product of dequantised operands.  Tolerance (stated by the benchmark spec): relative
Frobenius error <= 1e-3 for the fp32 epilogue; the bf16 output is compared with the bf16-rounded
oracle (bf16 rounding alone is ~1.7e-3 relative, above that bound)."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16, u8

pytestmark = pytest.mark.gpu

REL_FRO_TOL = 1e-3


def _quant_pair(M, N, K, seed, ec=True):
    tkq = mod("tk_quant_v5")
    x = o.make_activations(M, K, seed=seed)
    w = o.bf16_round((0.02 * np.random.default_rng(seed + 1).standard_normal((N, K))).astype(np.float32))
    qx = tkq.tk_quantize_for_gemm(to_dev_bf16(x), False, ec)
    qw = tkq.tk_quantize_for_gemm(to_dev_bf16(w), False, ec)
    return x, w, qx, qw


def _oracle_product(qx, qw, M, N, K):
    a_sc = o.unswizzle_scales(u8(qx[1]), M, K // 16)
    b_sc = o.unswizzle_scales(u8(qw[1]), N, K // 16)
    return o.nvfp4_gemm_fp32(u8(qx[0]), a_sc, qx[4].item(), u8(qw[0]), b_sc, qw[4].item())


# (256, 384, 512) and (128, 128, 256): N an odd multiple of 128 (half-empty last column tile) on both kernels;
# (2048, 9472, 512) and (4096, 4096, 256): several tiles per CTA pair, so that the accumulator alternates between its
# two tensor-memory positions and, with one K stage per tile, the epilogue is what the MMA thread waits for
@pytest.mark.parametrize("shape", [(128, 256, 256), (128, 256, 1024), (256, 512, 512), (384, 768, 2304),
                                   (1024, 1024, 4096), (256, 384, 512), (128, 128, 256), (2048, 9472, 512),
                                   (4096, 4096, 256)])
def test_nvfp4_gemm_fp32_and_bf16(shape):
    gemm = mod("tk_gemm_c")
    M, N, K = shape
    x, w, qx, qw = _quant_pair(M, N, K, seed=M + N + K)
    ref = _oracle_product(qx, qw, M, N, K)
    d32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], qw[0], qw[1], qw[4], d32)
    d16 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], qw[0], qw[1], qw[4], d16)
    torch.cuda.synchronize()
    assert_status_ok()
    got = d32.cpu().numpy()
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= REL_FRO_TOL, f"fp32 epilogue rel-Frobenius {rel}"
    assert rel < 1e-5
    got16 = d16.float().cpu().numpy()
    ref16 = o.bf16_round(ref)
    # accumulation-order differences may flip a bf16 rounding by one ulp in rare entries
    mism = (got16 != ref16)
    assert mism.mean() < 2e-3
    assert np.abs(got16 - ref16).max() <= np.abs(ref16).max() * 2.0 ** -7
    # and it approximates the un-quantised product like the reference's release gate requires
    full = x.astype(np.float64) @ w.astype(np.float64).T
    rel_q = np.linalg.norm(got - full) / np.linalg.norm(full)
    assert rel_q < 0.25


def test_backward_gemms_from_column_operands():
    """dgrad dX = dY . W (row operand of dY x column operand of W) and wgrad dW = dY^T . X (column operands of
    both): the column-wise packs feed the same GEMM; checked against the oracle's dequantised products."""
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    M, N, K = 512, 256, 768          # X [M,K], W [N,K], dY [M,N]
    x = o.make_activations(M, K, seed=1)
    w = o.bf16_round((0.02 * np.random.default_rng(2).standard_normal((N, K))).astype(np.float32))
    dy = o.bf16_round((1e-3 * np.random.default_rng(3).standard_normal((M, N))).astype(np.float32))
    qx, qw, qdy = (tkq.tk_quantize_for_gemm(to_dev_bf16(t), True, False) for t in (x, w, dy))
    rx, rw, rdy = (o.nvfp4_quantize_for_gemm(t, True, False) for t in (x, w, dy))
    # dgrad: [M,N] row operand of dY  x  column operand of W ([K, N/2])  ->  [M,K]
    dx = torch.empty((M, K), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qdy[0], qdy[1], qdy[4], qw[2], qw[3], qw[5], dx)
    ref = o.nvfp4_gemm_fp32(rdy["row_fp4"], rdy["row_sc_logical"], rdy["sg"], rw["col_fp4"], rw["col_sc_logical"], rw["sg"])
    torch.cuda.synchronize()
    assert np.linalg.norm(dx.cpu().numpy() - ref) / np.linalg.norm(ref) <= REL_FRO_TOL
    full = dy.astype(np.float64) @ w.astype(np.float64)
    assert np.linalg.norm(dx.cpu().numpy() - full) / np.linalg.norm(full) < 0.25
    # wgrad: column operand of dY ([N, M/2])  x  column operand of X ([K, M/2])  ->  [N,K]
    dw = torch.empty((N, K), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qdy[2], qdy[3], qdy[5], qx[2], qx[3], qx[5], dw)
    ref = o.nvfp4_gemm_fp32(rdy["col_fp4"], rdy["col_sc_logical"], rdy["sg"], rx["col_fp4"], rx["col_sc_logical"], rx["sg"])
    torch.cuda.synchronize()
    assert np.linalg.norm(dw.cpu().numpy() - ref) / np.linalg.norm(ref) <= REL_FRO_TOL
    assert_status_ok()


def test_grouped_residual_and_batched_accum():
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    M, K, H = 256, 512, 512
    x = o.make_activations(M, K, seed=4)
    w1 = o.bf16_round((0.02 * np.random.default_rng(5).standard_normal((H, K))).astype(np.float32))
    w3 = o.bf16_round((0.05 * np.random.default_rng(6).standard_normal((H, K))).astype(np.float32))
    qx = tkq.tk_quantize_for_gemm(to_dev_bf16(x), False, True)
    q1 = tkq.tk_quantize_for_gemm(to_dev_bf16(w1), False, True)
    q3 = tkq.tk_quantize_for_gemm(to_dev_bf16(w3), False, True)
    # grouped: concatenated weights, one tensor scale per 256 rows, two outputs
    b = torch.cat([q1[0].view(torch.uint8), q3[0].view(torch.uint8)], 0)
    b_sc = torch.cat([q1[1].view(torch.uint8), q3[1].view(torch.uint8)], 0)
    b_sg = torch.cat([q1[4].expand(H // 256), q3[4].expand(H // 256)]).contiguous()
    h1 = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
    h3 = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
    gemm.nvfp4_grouped_gemm(qx[0], qx[1], qx[4], b, b_sc, b_sg, h1, h3)
    s1 = torch.empty_like(h1); s3 = torch.empty_like(h3)
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], q1[0], q1[1], q1[4], s1)
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], q3[0], q3[1], q3[4], s3)
    torch.cuda.synchronize()
    assert torch.equal(h1, s1) and torch.equal(h3, s3)
    # residual epilogue: D = bf16(bf16(acc*sg) + R)
    r = torch.randn((M, H), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    d = torch.empty_like(h1)
    gemm.nvfp4_gemm_residual(qx[0], qx[1], qx[4], q1[0], q1[1], q1[4], r, d)
    torch.cuda.synchronize()
    assert torch.equal(d, (s1.float() + r.float()).to(torch.bfloat16))
    # batched accumulate: sum of two products kept in fp32, rounded once
    acc = torch.empty_like(h1)
    gemm.nvfp4_batched_accum_gemm([qx[0], qx[0]], [qx[1], qx[1]], [qx[4], qx[4]], [q1[0], q3[0]], [q1[1], q3[1]],
                                  [q1[4], q3[4]], acc)
    # the oracle's summation order on the raw accumulators (fp32 epilogue with unit tensor scales): first term
    # multiplied, the second joined by one fused multiply-add, one bf16 rounding at the end
    one = torch.ones(1, device="cuda")
    r1 = torch.empty((M, H), dtype=torch.float32, device="cuda"); r3 = torch.empty_like(r1)
    gemm.nvfp4_gemm(qx[0], qx[1], one, q1[0], q1[1], one, r1)
    gemm.nvfp4_gemm(qx[0], qx[1], one, q3[0], q3[1], one, r3)
    torch.cuda.synchronize()
    scales = [np.float32(qx[4].item()) * np.float32(q1[4].item()), np.float32(qx[4].item()) * np.float32(q3[4].item())]
    want = o.bf16_round(o.nvfp4_batched_accum_f32([r1.cpu().numpy(), r3.cpu().numpy()], scales))
    assert np.array_equal(acc.float().cpu().numpy(), want)
    assert_status_ok()


@pytest.mark.parametrize("M,Ks", [(384, (512, 512)), (512, (256, 768, 512)), (256, (512, 256, 256, 512))])
def test_batched_accum_forms_against_the_oracle_order(M, Ks):
    """The chain of launches (M not a multiple of 256: one-CTA kernel, fp32 partial between launches) and the one-launch
    form (terms of different reduction widths, three and four terms) against the oracle's summation order applied to
    the raw accumulators of the single GEMMs."""
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    N = 512
    A, Asc, Asg, B, Bsc, Bsg, raws, scales = [], [], [], [], [], [], [], []
    one = torch.ones(1, device="cuda")
    for i, K in enumerate(Ks):
        x, w, qx, qw = _quant_pair(M, N, K, seed=300 + 7 * i + M)
        A.append(qx[0]); Asc.append(qx[1]); Asg.append(qx[4]); B.append(qw[0]); Bsc.append(qw[1]); Bsg.append(qw[4])
        r = torch.empty((M, N), dtype=torch.float32, device="cuda")
        gemm.nvfp4_gemm(qx[0], qx[1], one, qw[0], qw[1], one, r)
        raws.append(r)
        scales.append(np.float32(qx[4].item()) * np.float32(qw[4].item()))
    d = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    gemm.nvfp4_batched_accum_gemm(A, Asc, Asg, B, Bsc, Bsg, d)
    torch.cuda.synchronize()
    want = o.bf16_round(o.nvfp4_batched_accum_f32([r.cpu().numpy() for r in raws], scales))
    assert np.array_equal(d.float().cpu().numpy(), want)
    assert_status_ok()


@pytest.mark.parametrize("M", [256, 384])       # one launch over the column slices / chained launches over copies
def test_split_dgrad_sum_reads_the_slices_where_they_are(M):
    """nvfp4_split_dgrad_sum on the column concatenation that the three-stream gradient quantiser produces (own tensor
    scale per stream) against the reference's arithmetic for it (nvfp4_b200_gemm.cu:2466-2487): one GEMM per split on
    a contiguous copy of its slice into a bf16 matrix of its own, then Tensor.add_ left to right."""
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    splits, n_out = [512, 256, 256], 512
    rng = np.random.default_rng(M)
    grads = [to_dev_bf16(o.bf16_round((s_ * rng.standard_normal((M, d))).astype(np.float32))) for d, s_ in zip(splits, (1e-3, 3e-3, 5e-4))]
    q = tkq.tk_group_quantize_dim1_split3_for_gemm(*grads)
    a_cat, a_sc_cat, sg = q[5], q[6], q[2]
    ws = [tkq.tk_quantize_for_gemm(to_dev_bf16(o.bf16_round((0.02 * rng.standard_normal((n_out, d))).astype(np.float32))), False, True)
          for d in splits]
    b_sg_cat = torch.cat([w[4] for w in ws]).contiguous()
    a_sg_list = [sg.narrow(0, i, 1) for i in range(3)]
    d = torch.full((M, n_out), float("nan"), dtype=torch.bfloat16, device="cuda")
    gemm.nvfp4_split_dgrad_sum(a_cat, a_sc_cat, a_sg_list, [w[0] for w in ws], [w[1] for w in ws], b_sg_cat, splits, d)
    a_u8, sc_u8 = a_cat.view(torch.uint8), a_sc_cat.view(torch.uint8)
    A, Asc, off = [], [], 0
    for dd in splits:
        A.append(a_u8[:, off // 2:(off + dd) // 2].contiguous())
        Asc.append(sc_u8[:, off // 64:(off + dd) // 64, :].contiguous())
        off += dd
    want = torch.empty_like(d)
    for i in range(3):
        term = want if i == 0 else torch.empty_like(d)
        gemm.nvfp4_gemm(A[i], Asc[i], a_sg_list[i], ws[i][0], ws[i][1], ws[i][4], term)
        if i:
            want.add_(term)
    torch.cuda.synchronize()
    assert torch.equal(d, want)
    assert_status_ok()


def test_batched_accum_equals_the_reference_kernels_bytes():
    """nvfp4_batched_accum_gemm with 2, 3 and 4 terms against the output bytes of the reference's own kernel on the
    same operands (tests/golden/make_accum_golden.py recorded them on a B200): pins the fp32 summation order."""
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "nvfp4_accum_reference_golden.npz"))
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_accum_golden",
                                                  os.path.join(os.path.dirname(__file__), "golden", "make_accum_golden.py"))
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    gemm = mod("tk_gemm_c")
    terms = mk.make_terms(4)
    for n in (2, 3, 4):
        d = torch.empty(mk.M, mk.N, dtype=torch.bfloat16, device="cuda")
        gemm.nvfp4_batched_accum_gemm(*mk.split(terms[:n]), d)
        torch.cuda.synchronize()
        bits = d.view(torch.int16).cpu().numpy()
        assert np.array_equal(bits[::8], gold[f"rows_{n}"]), n
        assert hashlib.sha256(bits.tobytes()).digest() == gold[f"sha256_{n}"].tobytes(), n
    assert_status_ok()


@pytest.mark.parametrize("M", [256, 384])       # the two-CTA kernel and the one-CTA kernel
def test_grouped_gemm_with_rope_epilogue(M):
    """Fused QKV projection with the rotary embedding in the epilogue: the fp32 epilogue of the same GEMM gives the
    scaled accumulator the rotation starts from, so the three forms (heads of 64 without the intermediate bf16
    rounding; packed split and packed single-output with it) can be checked bit for bit against the oracle's
    rotation of that accumulator; V is the plain bf16 rounding."""
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    K, q_dim, k_dim, v_dim, seq = 512, 512, 256, 256, 128
    N = q_dim + k_dim + v_dim
    x, w, qx, qw = _quant_pair(M, N, K, seed=M + 17)
    b_sg = qw[4].expand(N // 256).contiguous()
    d32 = torch.empty((M, N), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], qw[0], qw[1], qw[4], d32)
    torch.cuda.synchronize()
    v = d32.cpu().numpy()
    rng = np.random.default_rng(3)
    for head, form in ((64, "live64"), (128, "split"), (128, "cat"), (256, "split"), (32, "cat")):
        ang = rng.uniform(0, 2 * np.pi, size=(seq, head // 2)).astype(np.float32)
        cs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)
        cs_d = torch.from_numpy(cs).cuda()
        dq = torch.full((M, q_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        dk = torch.full((M, k_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        dv = torch.full((M, v_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        if form == "live64":
            gemm.nvfp4_grouped_gemm_rope_live64(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, cs_d, seq)
            got = torch.cat([dq, dk, dv], dim=1)
        elif form == "split":
            gemm.nvfp4_grouped_gemm_rope_packed_split(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, cs_d, seq, head, head)
            got = torch.cat([dq, dk, dv], dim=1)
        else:
            got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            gemm.nvfp4_grouped_gemm_rope_packed_cat(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, got, cs_d, seq, head, head,
                                                    q_dim, k_dim)
        torch.cuda.synchronize()
        assert_status_ok()
        ref = o.rope_epilogue(v, cs, head, q_dim + k_dim, form != "live64")
        assert np.array_equal(got.float().cpu().numpy(), ref), form
        # and the rotation is a rotation: pair norms of Q are those of the un-rotated bf16 product (to rounding)
        plain = o.bf16_round(v[:, :q_dim]).astype(np.float64)
        rot = got[:, :q_dim].float().cpu().numpy().astype(np.float64)
        n0 = np.hypot(plain[:, 0::2], plain[:, 1::2])
        n1 = np.hypot(rot[:, 0::2], rot[:, 1::2])
        assert np.abs(n1 - n0).max() <= 2.0 ** -6 * n0.max()
    with pytest.raises(RuntimeError):
        gemm.nvfp4_grouped_gemm_rope_packed_split(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, cs_d, seq, 128, 64)
    with pytest.raises(RuntimeError):
        gemm.nvfp4_grouped_gemm_rope_live64(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, cs_d, 96)


def test_rope_epilogue_over_many_row_blocks():
    """More tiles than CTA pairs (16 x 12 tiles of 256 x 256): every pair works through a run of tiles that crosses
    from one row block into the next, so the per-row-block refill of the rotation table (and the hand-over between
    the two epilogue warps of a lane quadrant) is exercised; every output element is checked against the oracle's
    rotation of the fp32 epilogue of the same GEMM."""
    gemm = mod("tk_gemm_c")
    M, K, q_dim, k_dim, v_dim, seq = 4096, 256, 2048, 512, 512, 1024
    N = q_dim + k_dim + v_dim
    x, w, qx, qw = _quant_pair(M, N, K, seed=91)
    b_sg = qw[4].expand(N // 256).contiguous()
    d32 = torch.empty((M, N), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], qw[0], qw[1], qw[4], d32)
    torch.cuda.synchronize()
    v = d32.cpu().numpy()
    rng = np.random.default_rng(8)
    for head, form in ((128, "split"), (64, "live64")):
        ang = rng.uniform(0, 2 * np.pi, size=(seq, head // 2)).astype(np.float32)
        cs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)
        cs_d = torch.from_numpy(cs).cuda()
        dq = torch.full((M, q_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        dk = torch.full((M, k_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        dv = torch.full((M, v_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        if form == "live64":
            gemm.nvfp4_grouped_gemm_rope_live64(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, cs_d, seq)
        else:
            gemm.nvfp4_grouped_gemm_rope_packed_split(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, cs_d, seq, head, head)
        torch.cuda.synchronize()
        assert_status_ok()
        got = torch.cat([dq, dk, dv], dim=1).float().cpu().numpy()
        ref = o.rope_epilogue(v, cs, head, q_dim + k_dim, form != "live64")
        assert np.array_equal(got, ref), form


@pytest.mark.parametrize("M", [256, 128])
def test_grouped_gemm_silu_epilogue(M):
    """silu_dim: x / (1 + exp(-x)) on the first output columns in the epilogue (hardware __expf: one bf16 step against
    the oracle), the remaining columns the plain bf16 rounding; with the heads-of-64 rotation behind it."""
    gemm = mod("tk_gemm_c")
    K, N, silu_dim, seq = 512, 768, 256, 128
    x, w, qx, qw = _quant_pair(M, N, K, seed=M + 23)
    b_sg = qw[4].expand(N // 256).contiguous()
    d32 = torch.empty((M, N), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], qw[0], qw[1], qw[4], d32)
    d = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    gemm.nvfp4_grouped_gemm(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, d, None, None, silu_dim)
    torch.cuda.synchronize()
    assert_status_ok()
    v = d32.cpu().numpy()
    got = d.float().cpu().numpy()
    assert np.array_equal(got[:, silu_dim:], o.bf16_round(v[:, silu_dim:]))
    with np.errstate(over="ignore"):
        act = (v[:, :silu_dim] / (np.float32(1.0) + np.exp(-v[:, :silu_dim]).astype(np.float32))).astype(np.float32)
    ref = o.bf16_round(act)
    step = np.maximum(np.abs(ref), 2.0 ** -100) * 2.0 ** -7
    assert (np.abs(got[:, :silu_dim] - ref) <= step).all() and (got[:, :silu_dim] == ref).mean() > 0.99
    # SiLU, then the rotation of Q and K (heads of 64)
    rng = np.random.default_rng(5)
    ang = rng.uniform(0, 2 * np.pi, size=(seq, 32)).astype(np.float32)
    cs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)
    dq, dk, dv = (torch.empty((M, 256), dtype=torch.bfloat16, device="cuda") for _ in range(3))
    gemm.nvfp4_grouped_gemm_rope_live64(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, torch.from_numpy(cs).cuda(),
                                        seq, silu_dim)
    torch.cuda.synchronize()
    assert_status_ok()
    v2 = v.copy()
    v2[:, :silu_dim] = act
    ref2 = o.rope_epilogue(v2, cs, 64, 512, False)
    got2 = torch.cat([dq, dk, dv], dim=1).float().cpu().numpy()
    assert np.array_equal(got2[:, 512:], ref2[:, 512:]) and np.array_equal(got2[:, 256:512], ref2[:, 256:512])
    tol = np.maximum(np.abs(ref2[:, :256]), np.abs(act).max() * 2.0 ** -8) * 2.0 ** -6
    assert (np.abs(got2[:, :256] - ref2[:, :256]) <= tol).all()
