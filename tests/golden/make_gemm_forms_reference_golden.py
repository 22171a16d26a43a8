"""Records the outputs of the GEMM forms of the reference's OWN compiled ``_C`` module on packed operands.

Test infrastructure.  Needs one B200 and ``_tk_quant_v5`` + ``_C`` compiled by ``oracle/build_ref.sh <checkout> all``.
The GEMM kernels are pipelined tcgen05 kernels (mbarriers and cluster barriers only).  The operands are quantised by
the reference's optional-mode quantiser with data stochastic rounding (its round-to-nearest path runs a kernel with a
grid-wide barrier) and STORED in the fixture, so that the tests feed the same packed operands to this library:

  nvfp4_gemm, nvfp4_gemm_residual                          D [M, N] bf16
  nvfp4_grouped_gemm                                       Q / K / V outputs with one scale per 256-column tile of B
  nvfp4_grouped_gemm_rope_live64, ..._rope_packed_cat      rotary epilogue, heads of 64; single-output form, heads of 128
  nvfp4_batched_gemm                                       two independent products
  nvfp4_split_dgrad_sum                                    two column slices of one A, summed in fp32
  nvfp4_row_rms_reduce                                     inverse RMS from row partials
  nvfp4_quantize, fp32_to_fp4x2, fp4x2_to_fp32             the module's own tile quantiser and code conversions

    python tests/golden/make_gemm_forms_reference_golden.py   # writes tests/golden/nvfp4_gemm_forms_reference_golden.npz
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from tests.golden.make_misc_reference_golden import _load, normal, rope_table  # noqa: E402
from tests.golden.make_rmsnorm_bwd_kernel_golden import pack  # noqa: E402  (matrix -> SHA-256 + every eighth row)

SEED, SUBSEQ = 20261128, 13
M, K, N = 512, 512, 768                       # N = Q 256 + K 256 + V 256
SEQ = 128


def main():
    q, c = _load("_tk_quant_v5"), _load("_C")
    dev = torch.device("cuda", 0)
    t = lambda a: torch.from_numpy(a).to(torch.bfloat16).to(dev)
    u8 = lambda x: x.contiguous().view(torch.uint8).cpu().numpy()
    i16 = lambda x: x.view(torch.int16).cpu().numpy()
    quant = lambda x: q.tk_quantize_for_gemm_opt(x, False, True, True, False, "none", False, SEED, SUBSEQ, 448.0, "row")
    out = {}
    qa, qb = quant(t(normal(M, K, 600))), quant(t(normal(N, K, 601, 0.02)))
    qa2, qb2 = quant(t(normal(M, K, 602))), quant(t(normal(N, K, 603, 0.02)))
    for name, qq in (("a", qa), ("b", qb), ("a2", qa2), ("b2", qb2)):
        out[f"{name}.fp4"], out[f"{name}.sc"], out[f"{name}.sg"] = u8(qq[0]), u8(qq[1]), qq[4].cpu().numpy()
    bf = lambda m, n: torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    d = bf(M, N)
    c.nvfp4_gemm(qa[0], qa[1], qa[4], qb[0], qb[1], qb[4], d)
    pack(out, "gemm", i16(d))
    r = t(normal(M, N, 610, 0.5))
    c.nvfp4_gemm_residual(qa[0], qa[1], qa[4], qb[0], qb[1], qb[4], r, d)
    pack(out, "gemm_residual", i16(d))
    b_sg = torch.cat([qb[4] * s for s in (1.0, 0.5, 2.0)]).contiguous()      # one scale per 256-column tile
    out["b_sg_per_tile"] = b_sg.cpu().numpy()
    dq, dk, dv = bf(M, 256), bf(M, 256), bf(M, 256)
    c.nvfp4_grouped_gemm(qa[0], qa[1], qa[4], qb[0], qb[1], b_sg, dq, dk, dv)
    for nm, dd in (("q", dq), ("k", dk), ("v", dv)):
        pack(out, "grouped." + nm, i16(dd))
    cs64 = torch.from_numpy(rope_table(SEQ, 64, 620)).to(dev)
    c.nvfp4_grouped_gemm_rope_live64(qa[0], qa[1], qa[4], qb[0], qb[1], b_sg, dq, dk, dv, cs64, SEQ)
    for nm, dd in (("q", dq), ("k", dk), ("v", dv)):
        pack(out, "live64." + nm, i16(dd))
    cs128 = torch.from_numpy(rope_table(SEQ, 128, 621)).to(dev)
    c.nvfp4_grouped_gemm_rope_packed_cat(qa[0], qa[1], qa[4], qb[0], qb[1], b_sg, d, cs128, SEQ, 128, 128, 256, 256)
    pack(out, "packed_cat", i16(d))
    d1, d2 = bf(M, N), bf(M, N)
    c.nvfp4_batched_gemm([qa[0], qa2[0]], [qa[1], qa2[1]], [qa[4], qa2[4]], [qb[0], qb2[0]], [qb[1], qb2[1]], [qb[4], qb2[4]], [d1, d2])
    pack(out, "batched.0", i16(d1))
    pack(out, "batched.1", i16(d2))
    # split dgrad: A = one row-quantised [M, 512] whose column halves go with two weights [N, 256]
    wq = [quant(t(normal(N, 256, 630 + i, 0.02))) for i in range(2)]
    for i in range(2):
        out[f"w{i}.fp4"], out[f"w{i}.sc"], out[f"w{i}.sg"] = u8(wq[i][0]), u8(wq[i][1]), wq[i][4].cpu().numpy()
    a_sg_list = [qa[4], (qa[4] * 0.75).contiguous()]
    out["split.a_sg1"] = a_sg_list[1].cpu().numpy()
    b_sg_cat = torch.cat([wq[0][4], wq[1][4]]).contiguous()
    c.nvfp4_split_dgrad_sum(qa[0], qa[1], a_sg_list, [wq[0][0], wq[1][0]], [wq[0][1], wq[1][1]], b_sg_cat, [256, 256], d)
    pack(out, "split_dgrad_sum", i16(d))
    # helpers
    part = torch.from_numpy(np.abs(np.random.default_rng(640).standard_normal((M, 16))).astype(np.float32) * 300.0).to(dev)
    inv = torch.empty(M, dtype=torch.float32, device=dev)
    c.nvfp4_row_rms_reduce(part, inv, 4096, 1e-5)
    out["row_rms_reduce"] = inv.cpu().numpy()
    # the module's own tile quantiser (1 x 16 and 16 x 16 blocks) and the code conversions
    src = t(normal(256, 384, 660))
    for tag, two_d in (("tkq_1d", False), ("tkq_2d", True)):
        fp4 = torch.empty(256, 192, dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)
        sc = torch.empty(256 // 128, 384 // 64, 512, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        sg = torch.empty(1, dtype=torch.float32, device=dev)
        c.nvfp4_quantize(src, fp4, sc, sg, two_d)
        torch.cuda.synchronize()
        out[f"{tag}.fp4"], out[f"{tag}.sc"], out[f"{tag}.sg"] = u8(fp4), u8(sc), sg.cpu().numpy()
    f32 = torch.from_numpy((np.random.default_rng(661).standard_normal((64, 128)) * 3.0).astype(np.float32)).to(dev)
    codes = c.fp32_to_fp4x2(f32)
    out["fp32_to_fp4x2"] = u8(codes)
    out["fp4x2_to_fp32"] = c.fp4x2_to_fp32(codes).cpu().numpy()
    torch.cuda.synchronize()
    dst = os.environ.get("GEMM_FORMS_GOLDEN_OUT", os.path.join(HERE, "nvfp4_gemm_forms_reference_golden.npz"))
    np.savez_compressed(dst, **out)
    print(f"wrote {dst}: {len(out)} arrays, {os.path.getsize(dst)} bytes")


if __name__ == "__main__":
    main()
