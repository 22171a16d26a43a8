"""GPU parity of the MXFP4 path: quantisers bit-exact vs the oracle (all three exponent modes),
fused RMSNorm bit-exact given the GPU's inverse RMS, GEMM within 1e-3 relative Frobenius of the
oracle's product of dequantised operands (fp32 epilogue)."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16, u8

pytestmark = pytest.mark.gpu


def _check(out, ref):
    for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
        assert np.array_equal(u8(out[i]).reshape(ref[k].shape), ref[k]), k


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (1024, 4096)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_mxfp4_quantize_row_and_col(shape, mode):
    mxq = mod("mxfp4_quant_v4")
    x = o.make_activations(*shape, seed=sum(shape) + mode)
    x[0, :32] = 0.0
    out = mxq.mxfp4_quantize_row_and_col(to_dev_bf16(x), mode)
    torch.cuda.synchronize()
    assert tuple(out[1].shape) == (shape[0] // 128, shape[1] // 128, 32, 16)
    _check(out, o.mxfp4_quantize_row_and_col(x, mode))
    row = mxq.mxfp4_quantize_for_gemm(to_dev_bf16(x), mode)
    assert torch.equal(row[0].view(torch.uint8), out[0].view(torch.uint8)) and torch.equal(row[1], out[1])
    assert_status_ok()


def test_mxfp4_fused_rmsnorm_and_silu():
    mxq = mod("mxfp4_quant_v4")
    M, K = 512, 1024
    x = o.make_activations(M, K, seed=31)
    g = o.make_gamma(K, seed=32)
    out = mxq.mxfp4_fused_rmsnorm_quantize_row_and_col(to_dev_bf16(x), to_dev_bf16(g), 1e-5, 1)
    torch.cuda.synchronize()
    inv = out[4].cpu().numpy()
    assert np.abs(inv / o.rmsnorm_inv_rms(x, 1e-5) - 1).max() < 2e-6
    _check(out, o.mxfp4_quantize_row_and_col(o.rmsnorm_apply(x, inv, g), 1))
    tkq = mod("tk_quant_v5")
    h1 = o.bf16_round(np.random.default_rng(5).standard_normal((256, 512)).astype(np.float32))
    h3 = o.bf16_round(np.random.default_rng(6).standard_normal((256, 512)).astype(np.float32))
    out = mxq.mxfp4_fused_silu_mul_quantize_row_and_col(to_dev_bf16(h1), to_dev_bf16(h3), 1)
    h_gpu = tkq.tk_silu_mul_split_bf16(to_dev_bf16(h1), to_dev_bf16(h3)).float().cpu().numpy()
    torch.cuda.synchronize()
    _check(out, o.mxfp4_quantize_row_and_col(h_gpu, 1))
    assert_status_ok()


# (4096, 4096): 1024 chunks over 296 CTAs, so a CTA walks three or four chunks and every buffer of its ring is reused
@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (384, 1280), (4096, 4096)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_one_pass_swiglu_producers_equal_element_kernel_plus_quantiser(shape, mode, monkeypatch):
    """The one-pass producers (activation computed on the chunk in shared memory, no bf16 intermediate in HBM) give
    the bytes of the oracle's quantiser applied to the element kernels' bf16 outputs, and the bytes of the two-pass
    route of the same mirrors."""
    mxq, tkq = mod("mxfp4_quant_v4"), mod("tk_quant_v5")
    M, H = shape
    g = torch.Generator(device="cuda").manual_seed(M + H + mode)
    mk = lambda s: (s * torch.randn(M, H, device="cuda", generator=g)).to(torch.bfloat16)
    h1, h3, dh = mk(1.5), mk(1.0), mk(1e-3)
    h1[0, :32] = 0.0                                     # an all-zero block of h and of dh3
    dh[-1, -32:] = 0.0
    monkeypatch.setenv("FP4B200_MX_ONE_PASS", "1")
    fwd = mxq.mxfp4_fused_silu_mul_quantize_row_and_col(h1, h3, mode)
    bwd = mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col(dh, h3, h1, mode)
    monkeypatch.setenv("FP4B200_MX_ONE_PASS", "0")
    fwd2 = mxq.mxfp4_fused_silu_mul_quantize_row_and_col(h1, h3, mode)
    bwd2 = mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col(dh, h3, h1, mode)
    torch.cuda.synchronize()
    for a, b in zip(fwd + bwd, fwd2 + bwd2):
        assert a.shape == b.shape and torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    if M * H <= 1 << 20:
        h = tkq.tk_silu_mul_split_bf16(h1, h3).float().cpu().numpy()
        _check(fwd, o.mxfp4_quantize_row_and_col(h, mode))
        for i, t in enumerate(tkq.tk_silu_deriv_split_bf16(dh, h3, h1)):
            _check([x[i] for x in bwd], o.mxfp4_quantize_row_and_col(t.float().cpu().numpy(), mode))
    assert_status_ok()


# K = 384, 1152: an odd multiple of 128 (half-depth last K stage); N = 384: half-empty last column tile
@pytest.mark.parametrize("shape", [(128, 256, 256), (256, 512, 1024), (512, 768, 2304), (256, 384, 384), (128, 256, 1152),
                                   (2048, 4096, 640)])
def test_mxfp4_gemm(shape):
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    M, N, K = shape
    x = o.make_activations(M, K, seed=M + K)
    w = o.bf16_round((0.02 * np.random.default_rng(N).standard_normal((N, K))).astype(np.float32))
    qx = mxq.mxfp4_quantize_for_gemm(to_dev_bf16(x), 1)
    qw = mxq.mxfp4_quantize_for_gemm(to_dev_bf16(w), 1)
    d = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    gemm.mxfp4_gemm(qx[0], qx[1], qw[0], qw[1], d)
    d16 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    gemm.mxfp4_gemm(qx[0], qx[1], qw[0], qw[1], d16)
    torch.cuda.synchronize()
    assert_status_ok()
    ref = o.mxfp4_gemm_fp32(u8(qx[0]), o.unswizzle_scales(u8(qx[1]).reshape(M // 128, K // 128, 512), M, K // 32),
                            u8(qw[0]), o.unswizzle_scales(u8(qw[1]).reshape(N // 128, K // 128, 512), N, K // 32))
    got = d.cpu().numpy()
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-3 and rel < 1e-5, rel
    full = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.linalg.norm(got - full) / np.linalg.norm(full) < 0.25
    assert np.abs(d16.float().cpu().numpy() - o.bf16_round(ref)).max() <= np.abs(ref).max() * 2.0 ** -7


@pytest.mark.parametrize("M", [128, 256])
def test_mxfp4_split2_dgrad_onepass(M):
    """D = (A[:, :H] . B1^T + A[:, H:] . B2^T) / 36 in one launch: K segments with their own scale tensors
    and B operands; both GEMM kernels (M = 128 -> one-CTA kernel, M = 256 -> CTA pair)."""
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    H, N = 512, 256
    rng = np.random.default_rng(M)
    dh1 = o.bf16_round(rng.standard_normal((M, H)).astype(np.float32))
    dh3 = o.bf16_round((2.0 * rng.standard_normal((M, H))).astype(np.float32))
    w1 = o.bf16_round((0.02 * rng.standard_normal((N, H))).astype(np.float32))
    w3 = o.bf16_round((0.03 * rng.standard_normal((N, H))).astype(np.float32))
    q1, q3 = mxq.mxfp4_quantize_for_gemm(to_dev_bf16(dh1), 1), mxq.mxfp4_quantize_for_gemm(to_dev_bf16(dh3), 1)
    qw1, qw3 = mxq.mxfp4_quantize_for_gemm(to_dev_bf16(w1), 1), mxq.mxfp4_quantize_for_gemm(to_dev_bf16(w3), 1)
    a_full = torch.cat([q1[0].view(torch.uint8), q3[0].view(torch.uint8)], dim=1).contiguous()
    d = torch.empty((M, N), dtype=torch.float32, device="cuda")
    gemm.mxfp4_split2_dgrad_strided_onepass_gemm(a_full.view(torch.float4_e2m1fn_x2), [q1[1], q3[1]], [0, H // 2], [H // 2, H // 2],
                                                 [qw1[0], qw3[0]], [qw1[1], qw3[1]], d, -1)
    d16 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    gemm.mxfp4_split2_dgrad_strided_onepass_gemm(a_full.view(torch.float4_e2m1fn_x2), [q1[1], q3[1]], [0, H // 2], [H // 2, H // 2],
                                                 [qw1[0], qw3[0]], [qw1[1], qw3[1]], d16)
    torch.cuda.synchronize()
    r1, r3 = o.mxfp4_quantize_1d(dh1, 1), o.mxfp4_quantize_1d(dh3, 1)
    rw1, rw3 = o.mxfp4_quantize_1d(w1, 1), o.mxfp4_quantize_1d(w3, 1)
    # the oracle's product already carries the 1/36 of each term; the sum of the two is what one pass computes
    ref = (o.mxfp4_gemm_fp32(r1[0], r1[1], rw1[0], rw1[1]).astype(np.float64)
           + o.mxfp4_gemm_fp32(r3[0], r3[1], rw3[0], rw3[1]).astype(np.float64))
    got = d.cpu().numpy()
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel <= 1e-3 and rel < 1e-5, rel
    assert np.abs(d16.float().cpu().numpy() - o.bf16_round(ref.astype(np.float32))).max() <= np.abs(ref).max() * 2.0 ** -7
    with pytest.raises(RuntimeError):
        gemm.mxfp4_split2_dgrad_strided_onepass_gemm(a_full.view(torch.float4_e2m1fn_x2), [q1[1], q3[1]], [0, H // 2], [H // 2, H // 2],
                                                     [qw1[0]], [qw1[1]], d)
    assert_status_ok()


def test_launch_inplace_twins_fill_the_callers_tensors():
    """The *_launch_inplace functions write the same bytes into caller-owned tensors as their allocating twins
    return, and reject tensors of the wrong shape or dtype."""
    mxq = mod("mxfp4_quant_v4")
    M, H = 256, 384
    rng = np.random.default_rng(31)
    mk = lambda s: to_dev_bf16(o.bf16_round((s * rng.standard_normal((M, H))).astype(np.float32)))
    x, h3, dh = mk(1.0), mk(1.0), mk(1e-3)
    u8 = dict(dtype=torch.uint8, device="cuda")

    def outs(lead=()):
        return (torch.empty((*lead, M, H // 2), **u8).view(torch.float4_e2m1fn_x2), torch.empty((*lead, M // 128, H // 128, 32, 16), **u8),
                torch.empty((*lead, H, M // 2), **u8).view(torch.float4_e2m1fn_x2), torch.empty((*lead, H // 128, M // 128, 32, 16), **u8))

    for mode in (0, 1, 2):
        got = outs()
        assert mxq.mxfp4_quantize_row_and_col_launch_inplace(x, *got, mode) is None
        want = mxq.mxfp4_quantize_row_and_col(x, mode)
        got2 = outs()
        mxq.mxfp4_fused_silu_mul_quantize_row_and_col_launch_inplace(x, h3, *got2, mode)
        want2 = mxq.mxfp4_fused_silu_mul_quantize_row_and_col(x, h3, mode)
        got3 = outs((2,))
        mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col_launch_inplace(dh, h3, x, *got3, mode)
        want3 = mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col(dh, h3, x, mode)
        torch.cuda.synchronize()
        for g, w in ((got, want), (got2, want2), (got3, want3)):
            for a, b in zip(g, w):
                assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    bad = outs()
    with pytest.raises(RuntimeError):
        mxq.mxfp4_quantize_row_and_col_launch_inplace(x, bad[0], bad[1].view(M // 128, H // 128, 512), bad[2], bad[3], 1)
    with pytest.raises(RuntimeError):
        mxq.mxfp4_quantize_row_and_col_launch_inplace(x, bad[0].view(torch.uint8), bad[1], bad[2], bad[3], 1)
    assert_status_ok()


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (512, 1024)])
@pytest.mark.parametrize("data_sr,scale_sr", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_mxfp4_quantize_for_gemm_opt_stochastic(shape, data_sr, scale_sr, mode):
    """Codes and scale bytes of the stochastic-rounding row quantiser, bit for bit on the reference's random stream."""
    mxq = mod("mxfp4_quant_v4")
    x = o.make_activations(*shape, seed=sum(shape) + 3 * mode)
    x[1, 32:64] = 0.0
    seed, subseq = 0x1234_5678_9ABC, 77 + mode
    out = mxq.mxfp4_quantize_for_gemm_opt(to_dev_bf16(x), mode, data_sr, scale_sr, seed, subseq)
    torch.cuda.synchronize()
    fp4, sc, _ = o.mxfp4_quantize_for_gemm_opt(x, mode, data_sr, scale_sr, seed, subseq)
    assert np.array_equal(u8(out[0]), fp4)
    assert np.array_equal(u8(out[1]).reshape(sc.shape), sc)
    assert_status_ok()


def test_mxfp4_quantize_for_gemm_opt_without_flags_is_the_plain_quantiser_and_sr_is_unbiased():
    mxq = mod("mxfp4_quant_v4")
    M, K = 1024, 2048
    x = o.make_activations(M, K, seed=9)
    xd = to_dev_bf16(x)
    plain = mxq.mxfp4_quantize_for_gemm(xd, 1)
    same = mxq.mxfp4_quantize_for_gemm_opt(xd, 1, False, False, 1, 2)
    assert torch.equal(plain[0].view(torch.uint8), same[0].view(torch.uint8)) and torch.equal(plain[1], same[1])
    # data SR with the ceil scale of mode 1 never saturates: the dequantised tensor is unbiased
    out = mxq.mxfp4_quantize_for_gemm_opt(xd, 1, True, False, 11, 5)
    torch.cuda.synchronize()
    fp4, sc, e = o.mxfp4_quantize_for_gemm_opt(x, 1, True, False, 11, 5)
    assert np.array_equal(u8(out[0]), fp4)
    deq = o.mxfp4_dequantize(fp4, e)
    rn = o.mxfp4_dequantize(*o.mxfp4_quantize_1d(x, 1))
    assert abs((deq - x).mean()) < 4.0 * np.linalg.norm(deq - x) / (M * K)   # four standard errors of the mean
    assert np.linalg.norm(deq - x) < 1.7 * np.linalg.norm(rn - x)
    assert_status_ok()


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (384, 256)])
@pytest.mark.parametrize("data_sr,scale_sr", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("mode", [0, 1])
def test_mxfp4_quantize_row_and_col_opt_stochastic(shape, data_sr, scale_sr, mode):
    """Row + column launch with correlated rounding of the codes and Philox rounding of the scales, bit for bit,
    on the second call of a run (the invocation offset of 2^40 is part of the stream's base)."""
    mxq = mod("mxfp4_quant_v4")
    x = o.make_activations(*shape, seed=sum(shape) + mode)
    x[3, 64:96] = 0.0
    seed, subseq = 0xC0FFEE, 456
    mxq.mxfp4_set_forward_sr_invocation_count(1)
    out = mxq.mxfp4_quantize_row_and_col_opt(to_dev_bf16(x), mode, data_sr, scale_sr, seed, subseq)
    torch.cuda.synchronize()
    assert mxq.mxfp4_forward_sr_invocation_count() == 2
    _check(out, o.mxfp4_quantize_row_and_col_opt(x, mode, data_sr, scale_sr, seed, subseq + (1 << 40)))
    assert_status_ok()


def test_mxfp4_correlated_rounding_agrees_between_the_views_and_advances():
    """The property the reference's own test of this launch asserts (mxfp4_v4/test_correlated_dual_sr.py): with the
    same maximum in every row block and column block, the row codes equal the transposed column codes, and two
    calls in a row round differently."""
    mxq = mod("mxfp4_quant_v4")
    n = 512
    ri, ci = np.arange(n)[:, None], np.arange(n)[None, :]
    peak = (ri % 32) == (ci % 32)
    rng = np.random.default_rng(17)
    x = (0.2 + 0.5 * rng.random((n, n))).astype(np.float32) * np.where(rng.random((n, n)) < 0.5, -1.0, 1.0)
    x[peak] = 1.0
    xd = to_dev_bf16(o.bf16_round(x.astype(np.float32)))
    mxq.mxfp4_set_forward_sr_invocation_count(0)
    prev = None
    for _ in range(3):
        out = mxq.mxfp4_quantize_row_and_col_opt(xd, 0, True, False, 123, 456)
        row = o.unpack_fp4(u8(out[0]))
        col = o.unpack_fp4(u8(out[2])).T
        assert np.array_equal(row, col)
        assert torch.equal(out[1], out[3])
        if prev is not None:
            assert (row != prev).mean() > 0.01
        prev = row
    assert mxq.mxfp4_forward_sr_invocation_count() == 3
    # the same test's second bound: over 64 calls, whether an off-peak element rounds up to code 4 is uncorrelated
    # (|r| < 0.02) with the same event 2, 4 or 8 elements further along either axis
    xs = np.full((n, n), 0.3, dtype=np.float32)
    xs[peak] = 1.0
    xd = to_dev_bf16(o.bf16_round(xs))
    ups = []
    for _ in range(64):
        out = mxq.mxfp4_quantize_row_and_col_opt(xd, 0, True, False, 123, 456)
        ups.append((o.unpack_fp4(u8(out[0])) == 4) & ~peak)
    ups = np.stack(ups).astype(np.float32)
    worst = 0.0
    for dr, dc in ((0, 2), (2, 0), (0, 4), (4, 0), (0, 8), (8, 0)):
        valid = ~peak[: n - dr, : n - dc] & ~peak[dr:, dc:]
        a = ups[:, : n - dr, : n - dc][:, valid].ravel()
        b = ups[:, dr:, dc:][:, valid].ravel()
        a, b = a - a.mean(), b - b.mean()
        worst = max(worst, abs(float((a * b).mean() / (a.std() * b.std()))))
    assert worst < 0.02, worst
    assert_status_ok()


@pytest.mark.parametrize("block", [16, 32])
@pytest.mark.parametrize("sign", [False, True])
@pytest.mark.parametrize("data_sr,scale_sr", [(False, False), (True, False), (True, True)])
def test_mxfp4_quantize_for_gemm_opt_rht(block, sign, data_sr, scale_sr):
    mxq = mod("mxfp4_quant_v4")
    M, K = 256, 384
    x = o.make_activations(M, K, seed=block + 2 * sign)
    out = mxq.mxfp4_quantize_for_gemm_opt_rht(to_dev_bf16(x), 1, data_sr, scale_sr, block, sign, 99, 3)
    torch.cuda.synchronize()
    fp4, sc, _ = o.mxfp4_quantize_for_gemm_opt(x, 1, data_sr, scale_sr, 99, 3, block, sign)
    assert np.array_equal(u8(out[0]), fp4)
    assert np.array_equal(u8(out[1]).reshape(sc.shape), sc)
    assert_status_ok()


@pytest.mark.parametrize("variant,row_rht,col_rht", [("mxfp4_quantize_row_and_col_opt_rht", False, True),
                                                     ("mxfp4_quantize_row_and_col_opt_rht_both", True, True),
                                                     ("mxfp4_quantize_row_and_col_opt_rht_row_only", True, False)])
@pytest.mark.parametrize("block", [16, 32])
@pytest.mark.parametrize("data_sr,scale_sr,sign", [(False, False, True), (True, False, False), (True, True, True),
                                                   (False, False, False)])
def test_mxfp4_quantize_row_and_col_opt_rht_variants(variant, row_rht, col_rht, block, data_sr, scale_sr, sign):
    mxq = mod("mxfp4_quant_v4")
    M, K = 256, 384
    x = o.make_activations(M, K, seed=7 + block)
    mxq.mxfp4_set_forward_sr_invocation_count(2)
    out = getattr(mxq, variant)(to_dev_bf16(x), 0, data_sr, scale_sr, block, sign, 31, 5)
    torch.cuda.synchronize()
    advanced = data_sr or scale_sr or sign
    assert mxq.mxfp4_forward_sr_invocation_count() == (3 if advanced else 2)
    ref = o.mxfp4_quantize_row_and_col_opt(x, 0, data_sr, scale_sr, 31, 5 + ((2 << 40) if advanced else 0), block, sign,
                                           row_rht, col_rht)
    _check(out, ref)
    assert_status_ok()


def test_mxfp4_rht_is_orthogonal_on_the_dequantised_tensor():
    """Round to nearest behind a 32-point transform along K: the inverse transform of the dequantised codes is as
    close to the input as the plain quantiser's output (the transform spreads outliers, it loses nothing)."""
    mxq = mod("mxfp4_quant_v4")
    M, K = 512, 1024
    x = o.make_activations(M, K, seed=4)
    out = mxq.mxfp4_quantize_for_gemm_opt_rht(to_dev_bf16(x), 1, False, False, 32, True, 1, 1)
    torch.cuda.synchronize()
    e = o.unswizzle_scales(u8(out[1]).reshape(M // 128, K // 128, 512), M, K // 32)
    deq_t = o.mxfp4_dequantize(u8(out[0]), e)
    t = o._mx_rht_segments(x.reshape(M, K // 16, 16), 32, True).reshape(M, K)
    plain = o.mxfp4_dequantize(*o.mxfp4_quantize_1d(x, 1))
    assert np.linalg.norm(deq_t - t) / np.linalg.norm(t) < 1.05 * np.linalg.norm(plain - x) / np.linalg.norm(x)
    assert_status_ok()


def test_reserved_coordinates_drive_the_stochastic_quantiser():
    """mxfp4_sr_state.reserve() -> (seed, subsequence) -> quantiser: two reservations of one producer give two
    different roundings, each reproduced by the oracle from the pair alone (what a resumed run relies on)."""
    mxq, sr = mod("mxfp4_quant_v4"), mod("mxfp4_sr_state")
    key = sr.ffn_w2_grad_key("layers.0.ffn")
    st = sr.MXFP4SRState([key, sr.qkv_grad_key("layers.0.attn")], user_seed=2024, user_subsequence_base=0,
                         training_steps=2, gradient_accumulation_steps=1)
    x = o.make_activations(128, 256, seed=12)
    xd = to_dev_bf16(x)
    seen = []
    for _ in range(2):
        seed, sub = st.reserve(key)
        out = mxq.mxfp4_quantize_for_gemm_opt(xd, 1, True, False, seed, sub)
        torch.cuda.synchronize()
        fp4, sc, _ = o.mxfp4_quantize_for_gemm_opt(x, 1, True, False, seed, sub)
        assert np.array_equal(u8(out[0]), fp4)
        seen.append(fp4)
    assert (seen[0] != seen[1]).mean() > 0.01
    resumed = sr.MXFP4SRState(st.logical_keys, user_seed=2024, user_subsequence_base=0, training_steps=2,
                              gradient_accumulation_steps=1)
    resumed.load_state_dict(st.state_dict())
    assert resumed.reserve(key) == st.reserve(key)
    assert_status_ok()
