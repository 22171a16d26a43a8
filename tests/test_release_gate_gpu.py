"""The reference's release gate for this path (tools/check_fp4_runtime_numerics.py), run through the mirrors: 512^3,
inputs from the CUDA generator with the gate's seed, NVFP4 route (tk_quantize_for_gemm -> nvfp4_gemm) and MXFP4 route
(signed 32-point Hadamard quantiser -> mxfp4_gemm) against the bf16 matmul.  The thresholds are the gate's; the
values the reference recorded on its own kernels (release/gpu_gate_receipt.json:47-56) are compared as well."""
import math

import pytest
import torch

from tests.gpu_util import assert_status_ok, mod

pytestmark = pytest.mark.gpu

SHAPE, SEED = 512, 20260903
RECEIPT = {"nvfp4_v5": (0.16246938705444336, 0.9868103265762329, 1.000624179840088),
           "mxfp4_v4_signed_h32": (0.16712865233421326, 0.9859760403633118, 0.9949585199356079)}
# The same generator and seed give the same inputs, and the recorded metrics come back to the last float32 digit or
# two (measured differences: 1.5e-8 in rel_l2, 6e-8 in cosine, 0 to 6e-8 in the norm ratio).  One differing code in
# 262144 outputs' worth of operands moves rel_l2 by more than this bound.
RECEIPT_TOL = 1e-6


def _inputs():
    g = torch.Generator(device="cuda")
    g.manual_seed(SEED)
    scale = SHAPE ** -0.25
    lhs = (torch.randn((SHAPE, SHAPE), device="cuda", dtype=torch.float32, generator=g) * scale).to(torch.bfloat16).contiguous()
    rhs = (torch.randn((SHAPE, SHAPE), device="cuda", dtype=torch.float32, generator=g) * scale).to(torch.bfloat16).contiguous()
    return lhs, rhs


def _metrics(actual, reference):
    a, r = actual.float(), reference.float()
    rn = torch.linalg.vector_norm(r)
    vals = (float(torch.linalg.vector_norm(a - r) / rn),
            float(torch.nn.functional.cosine_similarity(a.flatten(), r.flatten(), dim=0)),
            float(torch.linalg.vector_norm(a) / rn))
    assert all(math.isfinite(v) for v in vals)
    return vals


def _gate(label, vals):
    rel_l2, cosine, norm_ratio = vals
    assert rel_l2 < 0.25 and cosine > 0.96 and 0.80 <= norm_ratio <= 1.20, (label, vals)
    want = RECEIPT[label]
    print(label, "measured", vals, "recorded", want)
    assert all(abs(v - w) < RECEIPT_TOL for v, w in zip(vals, want)), (label, vals, want)


def test_nvfp4_route_passes_the_release_gate():
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    lhs, rhs = _inputs()
    reference = lhs @ rhs.t()
    lq, rq = tkq.tk_quantize_for_gemm(lhs, True), tkq.tk_quantize_for_gemm(rhs, True)
    actual = torch.empty_like(reference)
    gemm.nvfp4_gemm(lq[0], lq[1], lq[4], rq[0], rq[1], rq[4], actual)
    torch.cuda.synchronize()
    _gate("nvfp4_v5", _metrics(actual, reference))
    assert_status_ok()


def test_mxfp4_signed_h32_route_passes_the_release_gate():
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    lhs, rhs = _inputs()
    reference = lhs @ rhs.t()
    lq = mxq.mxfp4_quantize_for_gemm_opt_rht(lhs, 1, False, False, 32, True, 1234, 0)
    rq = mxq.mxfp4_quantize_for_gemm_opt_rht(rhs, 1, False, False, 32, True, 1234, 0)
    actual = torch.empty_like(reference)
    gemm.mxfp4_gemm(lq[0], lq[1], rq[0], rq[1], actual)
    torch.cuda.synchronize()
    _gate("mxfp4_v4_signed_h32", _metrics(actual, reference))
    assert_status_ok()


def test_correlated_rounding_reproduces_the_recorded_spatial_correlation():
    """The behaviour gate next to the two routes (mxfp4_v4/test_correlated_dual_sr.py; recorded maximum spatial
    correlation 0.001073, release/gpu_gate_receipt.json:59-62): 512 x 512 of 0.3 with 1.0 where row % 32 == col % 32,
    64 stochastic row + column launches from a fresh invocation counter with seed 123 / subsequence 456.  The two
    views agree, the rounding changes from call to call, and the correlation statistic equals the recorded one."""
    mxq = mod("mxfp4_quant_v4")
    n = 512
    ri = torch.arange(n, device="cuda")[:, None]
    ci = torch.arange(n, device="cuda")[None, :]
    peak = (ri % 32) == (ci % 32)
    values = torch.full((n, n), 0.3, device="cuda", dtype=torch.bfloat16)
    values[peak] = 1.0

    def unpack(t):
        p = t.view(torch.uint8)
        return torch.stack((p & 0x0F, p >> 4), dim=-1).reshape(p.shape[0], -1)

    mxq.mxfp4_set_forward_sr_invocation_count(0)
    samples, prev, change = [], None, []
    for _ in range(64):
        out = mxq.mxfp4_quantize_row_and_col_opt(values, 0, True, False, 123, 456)
        row, col = unpack(out[0]), unpack(out[2]).T.contiguous()
        assert torch.equal(row, col)
        if prev is not None:
            change.append(float((row != prev).float().mean()))
        prev = row
        samples.append((row == 4) & ~peak)
    assert sum(change) / len(change) > 0.01
    s = torch.stack(samples)

    def corr(a, b):
        a, b = a.float(), b.float()
        a, b = a - a.mean(), b - b.mean()
        return float((a * b).mean() / (a.std(unbiased=False) * b.std(unbiased=False)))

    worst = 0.0
    for dr, dc in ((0, 2), (2, 0), (0, 4), (4, 0), (0, 8), (8, 0)):
        valid = ~peak[: n - dr, : n - dc] & ~peak[dr:, dc:]
        worst = max(worst, abs(corr(s[:, : n - dr, : n - dc][:, valid], s[:, dr:, dc:][:, valid])))
    print("max spatial correlation", worst, "recorded 0.001073")
    assert worst < 0.02
    assert abs(worst - 0.001073) < 1e-6
    assert_status_ok()
