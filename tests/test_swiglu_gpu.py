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


def test_short_division_equals_the_general_one_for_every_bf16_input():
    """The element arithmetic divides by d = 1 + __expf(-x) with a reciprocal estimate, one Newton step and one
    corrected product wherever |x| < 64.  x is a bf16: all its patterns are compared on the device with the general
    IEEE division (x / d for SiLU, 1 / d for its derivative)."""
    lib = mod("_lib")
    out = torch.full((2,), 7, dtype=torch.int32, device="cuda")
    lib.call("fp4b200_selftest_silu_division", out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert out.tolist() == [0, 0]
    assert_status_ok()


def test_elements_outside_the_short_divisions_range():
    """Vectors that hold an element with |x| >= 64, an infinity or a NaN take the general division: the products
    keep the IEEE results there (silu(-100) = -0, silu(+inf) = +inf, sigmoid(-inf) = 0), -0 keeps its sign, and the
    neighbours in the same vector are the values they have in a vector of their own."""
    tkq = mod("tk_quant_v5")
    M, H = 128, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    h1 = (2.0 * torch.randn(M, H, device="cuda", generator=g)).to(torch.bfloat16)
    h3 = torch.randn(M, H, device="cuda", generator=g).to(torch.bfloat16)
    dh = (1e-3 * torch.randn(M, H, device="cuda", generator=g)).to(torch.bfloat16)
    plain = tkq.tk_silu_mul_split_bf16(h1, h3)
    d1p, d3p = tkq.tk_silu_deriv_split_bf16(dh, h3, h1)
    special = [-100.0, 100.0, 64.0, -64.0, -87.5, float("inf"), float("-inf"), float("nan"), -0.0, 63.75]
    h1s = h1.clone()
    for i, v in enumerate(special):
        h1s[i, 8 * i + 3] = v                                 # one special value per row, in vector 8*i .. 8*i+7
    h3s = h3.clone()
    h3s[:len(special)] = h3s[:len(special)].abs() + 1.0       # positive multipliers: signs of zeros are readable
    plain_s = tkq.tk_silu_mul_split_bf16(h1, h3s)
    got = tkq.tk_silu_mul_split_bf16(h1s, h3s)
    d1, d3 = tkq.tk_silu_deriv_split_bf16(dh, h3, h1s)
    torch.cuda.synchronize()
    mask = torch.zeros(M, H, dtype=torch.bool, device="cuda")
    for i in range(len(special)):
        mask[i, 8 * i + 3] = True
    same = lambda a, b: torch.equal(a.view(torch.int16)[~mask], b.view(torch.int16)[~mask])
    assert same(got, plain_s) and same(d1, d1p) and same(d3, d3p)
    at = lambda t, i: t[i, 8 * i + 3].float().item()
    bits = lambda t, i: t[i, 8 * i + 3].view(torch.int16).item() & 0xFFFF
    rb = lambda v: torch.tensor(v, dtype=torch.float32).to(torch.bfloat16).float().item()
    assert bits(got, 0) == 0x8000 and at(got, 1) == rb(100.0 * at(h3s, 1))      # silu(-100) = -0, silu(100) = 100
    assert at(got, 5) == float("inf") and np.isnan(at(got, 7))
    assert np.isnan(at(got, 6))                                                   # -inf / inf
    assert bits(got, 8) == 0x8000                                                 # -0 stays -0
    assert at(d3, 0) == 0.0 and at(d1, 0) == 0.0                                  # sigmoid(-100) = 0 exactly
    assert at(got, 9) == rb(63.75 * at(h3s, 9))                                   # silu(63.75) = 63.75 in fp32
    assert_status_ok()
