"""GPU parity of the SwiGLU producers.  The GPU evaluates exp with the hardware approximation
(__expf), so the bf16 products are compared with the oracle to one bf16 ulp, and the quantisation is
checked bit-exactly GIVEN the GPU's bf16 product (the part that is reproducible on a CPU)."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16, u8

pytestmark = pytest.mark.gpu


def _ulp_close(got, ref):
    """|got-ref| <= one bf16 ulp of the larger magnitude (plus a tiny absolute floor)."""
    mag = np.maximum(np.abs(got), np.abs(ref))
    ulp = np.maximum(mag * 2.0 ** -7, 1e-30)
    return np.abs(got - ref) <= ulp


def _inputs(M, H, seed):
    rng = np.random.default_rng(seed)
    h1 = o.bf16_round(rng.standard_normal((M, H)).astype(np.float32) * 2.0)
    h3 = o.bf16_round(rng.standard_normal((M, H)).astype(np.float32))
    dh = o.bf16_round(rng.standard_normal((M, H)).astype(np.float32) * 1e-3)
    return h1, h3, dh


@pytest.mark.parametrize("shape", [(128, 128), (256, 1024), (512, 3584)])
def test_silu_quantize_split(shape):
    tkq = mod("tk_quant_v5")
    M, H = shape
    h1, h3, _ = _inputs(M, H, seed=M + H)
    out = tkq.tk_silu_quantize_split_for_gemm(to_dev_bf16(h1), to_dev_bf16(h3))
    torch.cuda.synchronize()
    h_gpu = out[8].float().cpu().numpy()
    assert _ulp_close(h_gpu, o.silu_mul(h1, h3)).all()
    assert np.array_equal(tkq.tk_silu_mul_split_bf16(to_dev_bf16(h1), to_dev_bf16(h3)).float().cpu().numpy(), h_gpu)
    ref = o.nvfp4_quantize_for_gemm(h_gpu, True, True)
    assert out[6].item() == ref["amax"] and out[4].item() == ref["sg"]
    for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
        assert np.array_equal(u8(out[i]).reshape(ref[k].shape), ref[k]), k
    assert_status_ok()


@pytest.mark.parametrize("ec", [True, False])
def test_silu_deriv_quantize_split_opt(ec):
    tkq = mod("tk_quant_v5")
    M, H = 256, 1024
    h1, h3, dh = _inputs(M, H, seed=9)
    out = tkq.tk_silu_deriv_quantize_split_for_gemm_opt(to_dev_bf16(dh), to_dev_bf16(h3), to_dev_bf16(h1), True, ec,
                                                        False, False, "none")
    torch.cuda.synchronize()
    assert len(out) == 15
    r1, r3 = o.silu_deriv(dh, h3, h1)
    for idx, ref_val, base in ((13, r1, 0), (14, r3, 6)):
        g = out[idx].float().cpu().numpy()
        assert _ulp_close(g, ref_val).mean() > 0.9999   # fused multiply-add contraction may move a last bit
        assert np.abs(g - ref_val).max() <= 2.0 ** -6 * np.abs(ref_val).max()
        ref = o.nvfp4_quantize_for_gemm(g, True, ec)
        for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
            assert np.array_equal(u8(out[base + i]).reshape(ref[k].shape), ref[k]), (idx, k)
        assert out[base + 4].item() == ref["sg"] and out[base + 5].item() == ref["sg"]
    with pytest.raises(RuntimeError):
        tkq.tk_silu_deriv_quantize_split_for_gemm_opt(to_dev_bf16(dh), to_dev_bf16(h3), to_dev_bf16(h1), True, ec, False,
                                                      False, "col")
    out16 = tkq.tk_silu_deriv_quantize_split_for_gemm(to_dev_bf16(dh), to_dev_bf16(h3), to_dev_bf16(h1))
    torch.cuda.synchronize()
    assert len(out16) == 16 and out16[5].item() == 0.0
    assert_status_ok()
