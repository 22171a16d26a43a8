"""Seeded random shapes (multiples of the kernels' granularity, up to a few thousand on a side) through the
producers and the GEMMs: bytes against the oracle, products against the oracle's product.  The parametrised
tests elsewhere pick their shapes by hand; this walks ones nobody picked, including thin and wide matrices that
leave most CTAs without work or give a CTA a single chunk."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16, u8

pytestmark = pytest.mark.gpu

_rng = np.random.default_rng(20261125)
_QUANT_SHAPES = sorted({(int(128 * _rng.integers(1, 9)), int(128 * _rng.integers(1, 17))) for _ in range(14)}
                       | {(128, 2048), (1024, 128)})
_GEMM_SHAPES = sorted({(int(128 * _rng.integers(1, 7)), int(256 * _rng.integers(1, 5)), int(256 * _rng.integers(1, 9)))
                       for _ in range(10)})


def _operands_equal(out, ref):
    for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
        assert np.array_equal(u8(out[i]).reshape(ref[k].shape), ref[k]), k


@pytest.mark.parametrize("shape", _QUANT_SHAPES)
def test_quantisers_on_random_shapes(shape):
    tkq, mxq = mod("tk_quant_v5"), mod("mxfp4_quant_v4")
    M, K = shape
    seed = M * 31 + K
    x = o.make_activations(M, K, seed=seed)
    xd = to_dev_bf16(x)
    ec = bool(seed & 1)
    out = tkq.tk_quantize_for_gemm(xd, True, ec)
    torch.cuda.synchronize()
    _operands_equal(out, o.nvfp4_quantize_for_gemm(x, True, ec))
    # fused RMSNorm + quantise with the inverse RMS computed on the CPU: bit-exact end to end
    g = o.make_gamma(K, seed=seed + 1)
    inv = o.rmsnorm_inv_rms(x, 1e-5)
    fused = tkq.tk_fused_norm_quantize_from_inv_rms(xd, to_dev_bf16(g), torch.from_numpy(inv).cuda(), False, True)
    torch.cuda.synchronize()
    _operands_equal(fused, o.nvfp4_fused_norm_quantize(x, g, 1e-5, inv_rms=inv))
    # and with the GPU's own statistics: inverse RMS to hardware rsqrt accuracy, bytes exact given it
    own = tkq.tk_fused_norm_quantize(xd, to_dev_bf16(g), 1e-5, False, True)
    torch.cuda.synchronize()
    inv_gpu = own[5].cpu().numpy()
    assert np.abs(inv_gpu / inv - 1).max() < 2e-6
    _operands_equal(own, o.nvfp4_fused_norm_quantize(x, g, 1e-5, inv_rms=inv_gpu))
    mode = seed % 3
    mx = mxq.mxfp4_quantize_row_and_col(xd, mode)
    torch.cuda.synchronize()
    _operands_equal(mx, o.mxfp4_quantize_row_and_col(x, mode))
    assert_status_ok()


@pytest.mark.parametrize("shape", _GEMM_SHAPES)
def test_gemms_on_random_shapes(shape):
    tkq, mxq, gemm, gmx = mod("tk_quant_v5"), mod("mxfp4_quant_v4"), mod("tk_gemm_c"), mod("tk_gemm_c_mx")
    M, N, K = shape
    seed = M + 7 * N + 13 * K
    x = o.make_activations(M, K, seed=seed)
    w = o.bf16_round((0.02 * np.random.default_rng(seed + 1).standard_normal((N, K))).astype(np.float32))
    xd, wd = to_dev_bf16(x), to_dev_bf16(w)
    qx, qw = tkq.tk_quantize_for_gemm(xd, False, True), tkq.tk_quantize_for_gemm(wd, False, True)
    d = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    gemm.nvfp4_gemm(qx[0], qx[1], qx[4], qw[0], qw[1], qw[4], d)
    mx, mw = mxq.mxfp4_quantize_for_gemm(xd, 1), mxq.mxfp4_quantize_for_gemm(wd, 1)
    dm = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    gmx.mxfp4_gemm(mx[0], mx[1], mw[0], mw[1], dm)
    torch.cuda.synchronize()
    assert_status_ok()
    ref = o.nvfp4_gemm_fp32(u8(qx[0]), o.unswizzle_scales(u8(qx[1]), M, K // 16), qx[4].item(),
                            u8(qw[0]), o.unswizzle_scales(u8(qw[1]), N, K // 16), qw[4].item())
    rel = np.linalg.norm(d.cpu().numpy() - ref) / np.linalg.norm(ref)
    assert rel <= 1e-3 and rel < 1e-5, rel
    refm = o.mxfp4_gemm_fp32(u8(mx[0]), o.unswizzle_scales(u8(mx[1]).reshape(M // 128, K // 128, 512), M, K // 32),
                             u8(mw[0]), o.unswizzle_scales(u8(mw[1]).reshape(N // 128, K // 128, 512), N, K // 32))
    relm = np.linalg.norm(dm.cpu().numpy() - refm) / np.linalg.norm(refm)
    assert relm <= 1e-3 and relm < 1e-5, relm
