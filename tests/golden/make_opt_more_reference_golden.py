"""Records outputs of three more barrier-free entry points of the reference's OWN ``_tk_quant_v5`` module.

Test infrastructure.  Needs one B200 and ``_tk_quant_v5`` compiled by ``oracle/build_ref.sh <checkout> quant``.

  tk_quantize_transpose        one launch of the tuned TMA kernel with GIVEN tensor maxima: round to nearest (both
                               scale rules), stochastic codes, stochastic scale bytes, row / column Hadamard forms,
                               row operand switched off (tk_quantize.cu:3807-3926)
  tk_fused_norm_quantize_opt   RMSNorm + row Hadamard + stochastic rounding: inverse RMS kernel, scans, tuned kernel with
                               the normalisation fused (:8465-8586; without stochastic rounding it takes a persistent
                               kernel with a grid-wide barrier: not run)
  tk_silu_deriv_quantize_split_for_gemm_opt   element kernel, dual maximum kernel, tuned kernel per tensor (:10063-10255)

    python tests/golden/make_opt_more_reference_golden.py    # writes tests/golden/nvfp4_opt_more_reference_golden.npz

Runs in ONE fresh process, cases in the order below (the module numbers its stochastic launches from 0).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import fp4_oracle as o  # noqa: E402
from tests.golden.make_misc_reference_golden import _load, grads, normal  # noqa: E402

SEED, SUBSEQ = 20261129, 17
SHAPE = (128, 256)

# tk_quantize_transpose: (name, stochastic, encode_centric, scale_sr, row_rht, col_rht, return_transpose, return_row)
TRANSPOSE_CASES = [
    ("rtn_ec", False, True, False, False, False, True, True),
    ("rtn_dc", False, False, False, False, False, True, True),
    ("rtn_ec_row_only", False, True, False, False, False, False, True),
    ("rtn_dc_col_only", False, False, False, False, False, True, False),
    ("rht_row_dc", False, False, False, True, False, True, True),
    ("rht_col_ec", False, True, False, False, True, True, True),
    ("sr_dc", True, False, False, False, False, True, True),
    ("sr_scale_ec", True, True, True, False, False, True, True),
    ("scale_only_dc", False, False, True, False, False, True, True),
]
# tk_fused_norm_quantize_opt: (name, encode_centric, data_sr, scale_sr)
NORM_CASES = [("norm_sr_ec", True, True, False), ("norm_sr_scale_dc", False, True, True), ("norm_scale_only_ec", True, False, True)]
# tk_silu_deriv_quantize_split_for_gemm_opt: (name, encode_centric, data_sr, scale_sr, rht_axes, data_sr_axes)
SPLIT2_CASES = [("split2_sr_both", True, True, False, "row", "both"), ("split2_sr_row", False, True, False, "row", "row"),
                ("split2_sr_col", True, True, False, "row", "col"), ("split2_scale_only", True, False, True, "row", "both"),
                ("split2_plain", True, False, False, "row", "both")]


def transpose_input(i):
    return grads(*SHAPE, 1000 + i) if TRANSPOSE_CASES[i][1] or TRANSPOSE_CASES[i][3] else o.make_activations(*SHAPE, seed=1000 + i)


def main():
    q = _load("_tk_quant_v5")
    dev = torch.device("cuda", 0)
    t = lambda a: torch.from_numpy(a).to(torch.bfloat16).to(dev)
    u8 = lambda x: x.contiguous().view(torch.uint8).cpu().numpy()
    out = {}
    for i, (name, sr, ec, ssr, rr, cr, rt, ret_row) in enumerate(TRANSPOSE_CASES):
        x = t(transpose_input(i))
        amax = x.float().abs().max().reshape(1).contiguous()          # the plain maximum for both operands
        state = torch.tensor([SEED, SUBSEQ + (i << 32)], dtype=torch.int64, device=dev)
        r = q.tk_quantize_transpose(x, amax, amax, rt, sr, ec, ssr, rr, cr, ret_row, state)
        torch.cuda.synchronize()
        for j in range(4):
            if r[j].numel():
                out[f"{name}.{j}"] = u8(r[j])
    M, K = SHAPE
    for i, (name, ec, sr, ssr) in enumerate(NORM_CASES):
        x, g = t(o.make_activations(M, K, seed=1100 + i)), t(o.make_gamma(K, seed=1110 + i))
        r = q.tk_fused_norm_quantize_opt(x, g, 1e-5, True, ec, sr, ssr, "row", False, SEED, SUBSEQ)
        torch.cuda.synchronize()
        for j in range(4):
            out[f"{name}.{j}"] = u8(r[j])
        out[f"{name}.sg_row"], out[f"{name}.sg_col"], out[f"{name}.inv_rms"] = r[4].cpu().numpy(), r[5].cpu().numpy(), r[6].cpu().numpy()
    for i, (name, ec, sr, ssr, rht, axes) in enumerate(SPLIT2_CASES):
        dh, h3, h1 = t(grads(M, K, 1200 + i)), t(normal(M, K, 1210 + i)), t(normal(M, K, 1220 + i, 2.0))
        r = q.tk_silu_deriv_quantize_split_for_gemm_opt(dh, h3, h1, True, ec, sr, ssr, rht, False, SEED, SUBSEQ, axes)
        torch.cuda.synchronize()
        for j in (0, 1, 2, 3, 6, 7, 8, 9):
            out[f"{name}.{j}"] = u8(r[j])
        for j in (4, 5, 10, 11, 12):
            out[f"{name}.{j}"] = r[j].cpu().numpy()
        out[f"{name}.dh1"], out[f"{name}.dh3"] = r[13].view(torch.int16).cpu().numpy(), r[14].view(torch.int16).cpu().numpy()
    dst = os.environ.get("OPT_MORE_GOLDEN_OUT", os.path.join(HERE, "nvfp4_opt_more_reference_golden.npz"))
    np.savez_compressed(dst, **out)
    print(f"wrote {dst}: {len(out)} arrays, {os.path.getsize(dst)} bytes")


if __name__ == "__main__":
    main()
