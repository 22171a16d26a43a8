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


@pytest.mark.parametrize("shape", [(128, 256, 256), (256, 512, 1024), (512, 768, 2304)])
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
