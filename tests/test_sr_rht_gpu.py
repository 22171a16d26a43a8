"""GPU parity of the stochastic-rounding / Hadamard ("opt") producers against the oracle, which replays the
reference's Philox stream order (same seed / offset convention) and a rounding model of
``cvt.rs.satfinite.e2m1x4.f32`` measured on the GPU.  Bytes must be identical."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16, u8

pytestmark = pytest.mark.gpu


def _cmp(out, ref, keys=("row_fp4", "row_sc", "col_fp4", "col_sc")):
    for i, k in enumerate(keys):
        if k in ref:
            got = u8(out[i]).reshape(ref[k].shape)
            assert np.array_equal(got, ref[k]), f"{k}: {(got != ref[k]).mean():.4f} of bytes differ"


CASES = [
    dict(data_sr=True, rht="none", sign=False, axes="both"),
    dict(data_sr=True, rht="none", sign=False, axes="row"),
    dict(data_sr=True, rht="none", sign=False, axes="col"),
    dict(data_sr=False, rht="row", sign=False, axes="both"),
    dict(data_sr=False, rht="col", sign=False, axes="both"),
    dict(data_sr=False, rht="both", sign=True, axes="both"),
    dict(data_sr=True, rht="col", sign=True, axes="both"),
    dict(data_sr=True, rht="both", sign=False, axes="col"),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("ec", [True, False])
def test_quantize_for_gemm_opt(case, ec):
    tkq = mod("tk_quant_v5")
    M, K = 256, 384
    x = o.make_activations(M, K, seed=17, scale=1e-3 if case["axes"] == "col" else 1.0)
    seed, subseq = 0x1234ABCD5678, 77
    tkq.tk_set_sr_invocation_count(3)
    out = tkq.tk_quantize_for_gemm_opt(to_dev_bf16(x), True, ec, case["data_sr"], False, case["rht"], case["sign"],
                                       seed, subseq, 448.0, case["axes"])
    torch.cuda.synchronize()
    ref, used = o.nvfp4_quantize_for_gemm_opt(x, True, ec, case["data_sr"], case["rht"], case["sign"], seed, subseq,
                                              case["axes"], invocation=3)
    _cmp(out, ref)
    assert out[4].item() == ref["row_sg"] and out[5].item() == ref["col_sg"]
    assert tkq.tk_sr_invocation_count() == 3 + used
    assert_status_ok()


def test_sr_axis_isolation_and_advancing_offsets():
    """Properties the reference's test_advancing_sr.py pins: row-only SR leaves the column bytes equal to
    round-to-nearest; two calls in a row use different offsets and so differ."""
    tkq = mod("tk_quant_v5")
    x = to_dev_bf16(o.make_activations(256, 256, seed=3))
    rn = tkq.tk_quantize_for_gemm(x, True, False)
    a = tkq.tk_quantize_for_gemm_opt(x, True, False, True, False, "none", False, 11, 0, 448.0, "row")
    b = tkq.tk_quantize_for_gemm_opt(x, True, False, True, False, "none", False, 11, 0, 448.0, "row")
    torch.cuda.synchronize()
    assert torch.equal(a[2].view(torch.uint8), rn[2].view(torch.uint8))
    assert torch.equal(a[3].view(torch.uint8), rn[3].view(torch.uint8))
    assert not torch.equal(a[0].view(torch.uint8), rn[0].view(torch.uint8))
    assert not torch.equal(a[0].view(torch.uint8), b[0].view(torch.uint8))
    # unbiasedness: mean dequantised SR value is closer to x than the RTN bias bound
    assert_status_ok()


def test_sr_large_tensor_statistics():
    """Full 16384 x 4096 gradient-like tensor: SR codes dequantise to an (almost) unbiased estimate."""
    tkq = mod("tk_quant_v5")
    g = torch.Generator().manual_seed(5)
    x = (1e-3 * torch.randn(2048, 4096, generator=g)).to(torch.bfloat16)
    out = tkq.tk_quantize_for_gemm_opt(x.cuda(), False, False, True, False, "none", False, 99, 1, 448.0, "row")
    torch.cuda.synchronize()
    sc = o.unswizzle_scales(u8(out[1]), 2048, 4096 // 16)
    deq = o.nvfp4_dequantize(u8(out[0]), sc, out[4].item())
    xf = x.float().numpy()
    assert abs((deq - xf).mean()) < 2e-7
    assert np.linalg.norm(deq - xf) / np.linalg.norm(xf) < 0.25
    assert_status_ok()


@pytest.mark.parametrize("data_sr,scale_sr", [(True, False), (True, True), (False, True)])
def test_fused_norm_quantize_opt_row_rht_sr(data_sr, scale_sr):
    tkq = mod("tk_quant_v5")
    M, K = 256, 512
    x = o.make_activations(M, K, seed=41)
    g = o.make_gamma(K, seed=42)
    tkq.tk_set_sr_invocation_count(0)
    out = tkq.tk_fused_norm_quantize_opt(to_dev_bf16(x), to_dev_bf16(g), 1e-5, True, False, data_sr, scale_sr, "row",
                                         False, 7, 9)
    torch.cuda.synchronize()
    inv = out[6].cpu().numpy()
    n = o.rmsnorm_apply(x, inv, g)
    row_amax = o.rht16_amax(n, True)
    col_amax = o.tensor_amax(n)
    ref = o.nvfp4_quantize_transpose_launch(n, row_amax, col_amax, True, data_sr, False, True, False, True, 7, 9,
                                            scale_sr=scale_sr)
    _cmp(out, ref)
    assert out[4].item() == o.nvfp4_global_decode_scale(row_amax)
    assert out[5].item() == o.nvfp4_global_decode_scale(col_amax)
    assert_status_ok()


@pytest.mark.parametrize("axes,data_sr,scale_sr", [("both", True, False), ("row", True, False), ("both", True, True),
                                                   ("row", True, True), ("both", False, True)])
def test_silu_deriv_opt_row_rht_sr(axes, data_sr, scale_sr):
    tkq = mod("tk_quant_v5")
    M, H = 256, 512
    rng = np.random.default_rng(8)
    h1 = o.bf16_round(rng.standard_normal((M, H)).astype(np.float32))
    h3 = o.bf16_round(rng.standard_normal((M, H)).astype(np.float32))
    dh = o.bf16_round(rng.standard_normal((M, H)).astype(np.float32) * 1e-3)
    tkq.tk_set_sr_invocation_count(5)
    out = tkq.tk_silu_deriv_quantize_split_for_gemm_opt(to_dev_bf16(dh), to_dev_bf16(h3), to_dev_bf16(h1), True, False,
                                                        data_sr, scale_sr, "row", False, 21, 4, axes)
    torch.cuda.synchronize()
    assert len(out) == 15 and tkq.tk_sr_invocation_count() == 7
    for base, idx, n in ((0, 13, 5), (6, 14, 6)):
        t = out[idx].float().cpu().numpy()
        row_amax, orig = o.rht16_amax(t, True), o.tensor_amax(t)
        off = 4 + n * (1 << 32)
        if axes == "both" or not data_sr:
            ref = o.nvfp4_quantize_transpose_launch(t, row_amax, orig, True, data_sr, False, True, False, True, 21, off,
                                                    scale_sr=scale_sr)
        else:
            ref = o.nvfp4_quantize_transpose_launch(t, row_amax, orig, False, True, False, True, False, True, 21, off,
                                                    scale_sr=scale_sr)
            ref.update(o.nvfp4_quantize_transpose_launch(t, row_amax, orig, True, False, False, True, False, False, 21, off,
                                                         scale_sr=scale_sr))
        _cmp(out[base:base + 4], ref)
        assert out[base + 4].item() == o.nvfp4_global_decode_scale(row_amax)
        assert out[base + 5].item() == o.nvfp4_global_decode_scale(orig)
    assert_status_ok()


SCALE_SR_CASES = [
    dict(data_sr=False, rht="none", sign=False, axes="both", rt=True),
    dict(data_sr=True, rht="none", sign=False, axes="both", rt=True),
    dict(data_sr=True, rht="none", sign=False, axes="row", rt=True),
    dict(data_sr=True, rht="none", sign=False, axes="col", rt=True),
    dict(data_sr=False, rht="none", sign=False, axes="both", rt=False),
    dict(data_sr=True, rht="col", sign=True, axes="both", rt=True),
]


@pytest.mark.parametrize("case", SCALE_SR_CASES)
@pytest.mark.parametrize("ec", [True, False])
def test_scale_stochastic_rounding(case, ec):
    """Stochastic rounding of the E4M3 scale bytes (one more random word per block, drawn before the block's data
    words), alone and together with data SR on both axes or one: bytes identical to the oracle's replay of the
    reference's stream with the measured model of ``cvt.rs.satfinite.e4m3x4.f32``.  No block of the input is all
    zero (there the reference, encode-centric, would draw one word fewer)."""
    tkq = mod("tk_quant_v5")
    M, K = 256, 384
    x = o.make_activations(M, K, seed=23)
    seed, subseq = 0xFEDCBA987, 5
    tkq.tk_set_sr_invocation_count(11)
    out = tkq.tk_quantize_for_gemm_opt(to_dev_bf16(x), case["rt"], ec, case["data_sr"], True, case["rht"], case["sign"],
                                       seed, subseq, 448.0, case["axes"])
    torch.cuda.synchronize()
    ref, used = o.nvfp4_quantize_for_gemm_opt(x, case["rt"], ec, case["data_sr"], case["rht"], case["sign"], seed, subseq,
                                              case["axes"], invocation=11, scale_sr=True)
    _cmp(out, ref)
    assert tkq.tk_sr_invocation_count() == 11 + used
    # the scale bytes do move: a good part of them differs from the round-to-nearest launch
    plain, _ = o.nvfp4_quantize_for_gemm_opt(x, case["rt"], ec, case["data_sr"], case["rht"], case["sign"], seed, subseq,
                                             case["axes"], invocation=11)
    assert (ref["row_sc"] != plain["row_sc"]).mean() > 0.05
    assert_status_ok()


def test_scale_sr_is_unbiased_on_a_large_tensor():
    """Decode-centric scale SR on 2 M blocks: the mean of the decoded scale bytes matches the mean of the unrounded
    scales far better than round-to-nearest's systematic offset allows it to."""
    tkq = mod("tk_quant_v5")
    M, K = 2048, 16384
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    out = tkq.tk_quantize_for_gemm_opt(x, False, False, False, True, "none", False, 99, 0, 448.0, "both")
    torch.cuda.synchronize()
    amax = x.float().abs().max().item()
    s_enc = np.float32(2688.0) / np.float32(amax)
    b = x.float().abs().view(M, K // 16, 16).amax(dim=-1).cpu().numpy()
    exact = b.astype(np.float64) / 6.0 * float(s_enc)
    sc = o.e4m3_decode(o.unswizzle_scales(u8(out[1]), M, K // 16)).astype(np.float64)
    rel = abs(sc.mean() - exact.mean()) / exact.mean()
    assert rel < 2e-4, rel
    assert_status_ok()
