"""GPU parity of the GEMM forms against the outputs of the reference's OWN compiled ``_C`` kernels on the same packed
operands (tests/golden/nvfp4_gemm_forms_reference_golden.npz, recorded by
tests/golden/make_gemm_forms_reference_golden.py on a B200; the operands are in the fixture): plain and residual GEMM,
grouped GEMM with per-tile scales, the rotary epilogues (heads of 64, three outputs; heads of 128, one output), two
batched products, the split dgrad sum over column slices, and the row-partial inverse RMS.  Bit-exact, no tolerance."""
import os

import numpy as np
import pytest
import torch

from tests.golden import make_gemm_forms_reference_golden as G
from tests.golden.make_misc_reference_golden import normal, rope_table
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16

pytestmark = pytest.mark.gpu

_PATH = os.path.join(os.path.dirname(__file__), "golden", "nvfp4_gemm_forms_reference_golden.npz")
GOLD = np.load(_PATH) if os.path.exists(_PATH) else None
_i16 = lambda t: t.view(torch.int16).cpu().numpy()


def _eq(key, got):
    """The fixture keeps a matrix as every eighth row (to say where a difference is) and the SHA-256 of all of it."""
    import hashlib
    a = np.ascontiguousarray(got)
    bad = int((a[::8] != GOLD[key + ".rows8"]).sum())
    assert bad == 0, f"{key}: {bad} values of the sampled rows differ from the reference kernel's"
    digest = np.frombuffer(hashlib.sha256(a.tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(digest, GOLD[key + ".sha256"]), f"{key}: the bytes outside the sampled rows differ"


def _operand(name, rows, k):
    fp4, e4m3 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
    return (torch.from_numpy(GOLD[name + ".fp4"]).cuda().view(fp4).view(rows, k // 2),
            torch.from_numpy(GOLD[name + ".sc"]).cuda().view(e4m3), torch.from_numpy(GOLD[name + ".sg"]).cuda())


@pytest.mark.skipif(GOLD is None, reason="fixture not recorded")
def test_gemm_forms_reproduce_the_reference_kernels_outputs():
    gemm = mod("tk_gemm_c")
    M, K, N, SEQ = G.M, G.K, G.N, G.SEQ
    a, b, a2, b2 = _operand("a", M, K), _operand("b", N, K), _operand("a2", M, K), _operand("b2", N, K)
    bf = lambda m, n: torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    d = bf(M, N)
    gemm.nvfp4_gemm(*a, *b, d)
    _eq("gemm", _i16(d))
    gemm.nvfp4_gemm_residual(*a, *b, to_dev_bf16(normal(M, N, 610, 0.5)), d)
    _eq("gemm_residual", _i16(d))
    b_sg = torch.from_numpy(GOLD["b_sg_per_tile"]).cuda()
    dq, dk, dv = bf(M, 256), bf(M, 256), bf(M, 256)
    gemm.nvfp4_grouped_gemm(*a, b[0], b[1], b_sg, dq, dk, dv)
    _eq("grouped.q", _i16(dq)); _eq("grouped.k", _i16(dk)); _eq("grouped.v", _i16(dv))
    cs64 = torch.from_numpy(rope_table(SEQ, 64, 620)).cuda()
    gemm.nvfp4_grouped_gemm_rope_live64(*a, b[0], b[1], b_sg, dq, dk, dv, cs64, SEQ)
    _eq("live64.q", _i16(dq)); _eq("live64.k", _i16(dk)); _eq("live64.v", _i16(dv))
    cs128 = torch.from_numpy(rope_table(SEQ, 128, 621)).cuda()
    gemm.nvfp4_grouped_gemm_rope_packed_cat(*a, b[0], b[1], b_sg, d, cs128, SEQ, 128, 128, 256, 256)
    _eq("packed_cat", _i16(d))
    d1, d2 = bf(M, N), bf(M, N)
    gemm.nvfp4_batched_gemm([a[0], a2[0]], [a[1], a2[1]], [a[2], a2[2]], [b[0], b2[0]], [b[1], b2[1]], [b[2], b2[2]], [d1, d2])
    _eq("batched.0", _i16(d1)); _eq("batched.1", _i16(d2))
    w = [_operand(f"w{i}", N, 256) for i in range(2)]
    a_sg_list = [a[2], torch.from_numpy(GOLD["split.a_sg1"]).cuda()]
    b_sg_cat = torch.cat([w[0][2], w[1][2]]).contiguous()
    gemm.nvfp4_split_dgrad_sum(a[0], a[1], a_sg_list, [w[0][0], w[1][0]], [w[0][1], w[1][1]], b_sg_cat, [256, 256], d)
    _eq("split_dgrad_sum", _i16(d))
    part = torch.from_numpy(np.abs(np.random.default_rng(640).standard_normal((M, 16))).astype(np.float32) * 300.0).cuda()
    inv = torch.empty(M, dtype=torch.float32, device="cuda")
    gemm.nvfp4_row_rms_reduce(part, inv, 4096, 1e-5)
    torch.cuda.synchronize()
    assert np.array_equal(inv.cpu().numpy(), GOLD["row_rms_reduce"])
    assert_status_ok()


@pytest.mark.skipif(GOLD is None or "tkq_1d.fp4" not in (GOLD.files if GOLD is not None else ()), reason="fixture not recorded")
def test_tile_quantiser_and_code_conversions_reproduce_the_reference_kernels_bytes():
    gemm = mod("tk_gemm_c")
    src = to_dev_bf16(normal(256, 384, 660))
    for tag, two_d in (("tkq_1d", False), ("tkq_2d", True)):
        fp4 = torch.empty(256, 192, dtype=torch.uint8, device="cuda").view(torch.float4_e2m1fn_x2)
        sc = torch.empty(2, 6, 512, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
        sg = torch.empty(1, dtype=torch.float32, device="cuda")
        gemm.nvfp4_quantize(src, fp4, sc, sg, two_d)
        torch.cuda.synchronize()
        for key, got in ((f"{tag}.fp4", fp4), (f"{tag}.sc", sc)):
            got = got.view(torch.uint8).cpu().numpy().reshape(-1)
            bad = int((got != GOLD[key].reshape(-1)).sum())
            assert bad == 0, f"{key}: {bad} of {got.size} bytes differ from the reference kernel's"
        assert sg.item() == GOLD[f"{tag}.sg"].reshape(-1)[0]
    f32 = torch.from_numpy((np.random.default_rng(661).standard_normal((64, 128)) * 3.0).astype(np.float32)).cuda()
    codes = gemm.fp32_to_fp4x2(f32)
    assert np.array_equal(codes.view(torch.uint8).cpu().numpy(), GOLD["fp32_to_fp4x2"])
    assert np.array_equal(gemm.fp4x2_to_fp32(codes).cpu().numpy(), GOLD["fp4x2_to_fp32"])
    assert_status_ok()
