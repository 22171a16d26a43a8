"""Records the output bytes of the reference's OWN sm_100a MXFP4 quantiser kernels on seeded inputs.

Test infrastructure.  Needs one B200 and the reference's ``mxfp4_quant_v4`` extension module compiled by
``oracle/build_ref.sh <checkout> mxquant`` into ``oracle/_ref/`` (the reference's sources are not needed at run time):

    python tests/golden/make_mx_reference_golden.py     # writes tests/golden/mxfp4_reference_kernels_golden.npz

No kernel of that module waits on another CTA (read in mxfp4_v4/tk_quantize.cu and mxfp4_v3_quantize.cuh: no
grid-wide counter or flag), so every entry point listed in CASES is called.  Inputs are regenerated from their seeds
by the tests (``make_inputs`` below), so the fixture holds outputs only.  Calls run in the order of CASES in ONE fresh
process.
"""
import glob
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import fp4_oracle as o  # noqa: E402

SEED, SUBSEQ = 20261126, 5 << 32
SHAPE = (256, 384)

# name -> (function, positional arguments after the tensors)
CASES = [
    ("rowcol_m0", "mxfp4_quantize_row_and_col", "x", (0,)),
    ("rowcol_m1", "mxfp4_quantize_row_and_col", "x", (1,)),
    ("rowcol_m2", "mxfp4_quantize_row_and_col", "x", (2,)),
    ("row_only_m1", "mxfp4_quantize_for_gemm", "x", (1,)),
    ("weight_2d", "mxfp4_quantize_weight_2d", "w", ()),
    ("rmsnorm_m1", "mxfp4_fused_rmsnorm_quantize_row_and_col", "x_gamma", (1e-5, 1)),
    ("silu_mul_m1", "mxfp4_fused_silu_mul_quantize_row_and_col", "h1_h3", (1,)),
    ("silu_mul_m0", "mxfp4_fused_silu_mul_quantize_row_and_col", "h1_h3", (0,)),
    ("silu_deriv_m1", "mxfp4_fused_silu_deriv_quantize_split2_row_and_col", "dh_h3_h1", (1,)),
    ("row_sr_data", "mxfp4_quantize_for_gemm_opt", "g", (1, True, False, SEED, SUBSEQ)),
    ("row_sr_scale", "mxfp4_quantize_for_gemm_opt", "g", (1, False, True, SEED, SUBSEQ)),
    ("row_sr_both", "mxfp4_quantize_for_gemm_opt", "g", (0, True, True, SEED, SUBSEQ)),
    ("rowcol_sr_data", "mxfp4_quantize_row_and_col_opt", "g", (1, True, False, SEED, SUBSEQ)),
    ("rowcol_sr_both", "mxfp4_quantize_row_and_col_opt", "g", (1, True, True, SEED, SUBSEQ)),
    ("row_rht16_sign", "mxfp4_quantize_for_gemm_opt_rht", "g", (1, False, False, 16, True, SEED, SUBSEQ)),
    ("row_rht32_sr", "mxfp4_quantize_for_gemm_opt_rht", "g", (1, True, False, 32, True, SEED, SUBSEQ)),
    ("rowcol_rht_col16", "mxfp4_quantize_row_and_col_opt_rht", "g", (1, False, False, 16, True, SEED, SUBSEQ)),
    ("rowcol_rht_col32_sr", "mxfp4_quantize_row_and_col_opt_rht", "g", (1, True, False, 32, True, SEED, SUBSEQ)),
    ("rowcol_rht_both16", "mxfp4_quantize_row_and_col_opt_rht_both", "g", (1, False, False, 16, True, SEED, SUBSEQ)),
    ("rowcol_rht_row_only16", "mxfp4_quantize_row_and_col_opt_rht_row_only", "g", (1, False, False, 16, True, SEED, SUBSEQ)),
    ("silu_deriv_combined_m1", "mxfp4_fused_silu_deriv_quantize_split2_row_and_col_strided_combined", "dh_h13",
     (SHAPE[1], SHAPE[1], 1)),
    ("silu_deriv_splitcols_m1", "mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols", "dh_h3_h1", (1,)),
    ("silu_mul_strided_m1", "mxfp4_fused_silu_mul_quantize_row_and_col_strided", "h13", (SHAPE[1], SHAPE[1], 1)),
    ("split2_m1", "mxfp4_quantize_split2_row_and_col", "g2", (1,)),
    ("split3_m1", "mxfp4_quantize_split3_row_and_col", "g3", (1,)),
    ("split3_m0", "mxfp4_quantize_split3_row_and_col", "g3", (0,)),
    ("nhsd_d64_m1", "mxfp4_quantize_nhsd_wo_row_and_col", "nhsd64", (1,)),
    ("nhsd_d128_m1", "mxfp4_quantize_nhsd_wo_row_and_col", "nhsd128", (1,)),
    ("col_only_m1", "mxfp4_quantize_col_only", "x", (1,)),
]


def make_inputs(kind, seed):
    """The seeded inputs of a case as float32 arrays of bf16 values; the tests call this too."""
    M, K = SHAPE
    rng = np.random.default_rng(seed)
    r = lambda s: o.bf16_round((s * rng.standard_normal((M, K))).astype(np.float32))
    if kind == "x":
        x = o.make_activations(M, K, seed=seed).copy()
        x[3, 32:64] = 0.0                      # an all-zero row block
        x[64:96, 7] = 0.0                      # an all-zero column block
        return (x,)
    if kind == "w":
        return (r(0.02),)
    if kind == "x_gamma":
        return (o.make_activations(M, K, seed=seed), o.make_gamma(K, seed=seed + 1))
    if kind == "h1_h3":
        return (r(2.0), r(1.0))
    if kind == "dh_h3_h1":
        return (r(1e-3), r(1.0), r(2.0))
    if kind == "g":
        return (r(1e-3),)
    if kind in ("g2", "g3"):      # gradients of a fused projection's outputs: different widths, the same rows
        widths = (K, 128) if kind == "g2" else (256, 128, K)
        return tuple(o.bf16_round((1e-3 * 4.0 ** i * rng.standard_normal((M, w))).astype(np.float32)) for i, w in enumerate(widths))
    if kind in ("nhsd64", "nhsd128"):   # attention output [B, H, S, D]
        shape = (2, 4, 128, 64) if kind == "nhsd64" else (1, 3, 256, 128)
        return (o.bf16_round(rng.standard_normal(shape).astype(np.float32)),)
    if kind == "h13":
        return (np.concatenate([r(2.0), r(1.0)], axis=1),)
    if kind == "dh_h13":       # the packed gate|up activation: h1 in the left half, h3 in the right
        return (r(1e-3), np.concatenate([r(2.0), r(1.0)], axis=1))
    raise ValueError(kind)


def load_reference_module():
    paths = glob.glob(os.path.join(ROOT, "oracle", "_ref", "mxfp4_quant_v4*.so"))
    if not paths:
        raise SystemExit("oracle/_ref/mxfp4_quant_v4*.so is missing: run oracle/build_ref.sh <reference checkout> mxquant")
    spec = importlib.util.spec_from_file_location("mxfp4_quant_v4", paths[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


GEMM_SHAPES = [(256, 256, 512), (256, 512, 1280)]   # M, N, K
ONEPASS = (256, 256, 512)                           # M, N, width of each of the two splits


def gemm_operands(shape, seed):
    """bf16-valued float32 A [M, K] and B [N, K] of a GEMM case; the tests call this too."""
    M, N, K = shape
    rng = np.random.default_rng(seed)
    return (o.bf16_round(rng.standard_normal((M, K)).astype(np.float32)),
            o.bf16_round((0.02 * rng.standard_normal((N, K))).astype(np.float32)))


def combined_inputs():
    """dh [M, w] and the packed gate|up activation [M, 2w] of the combined-producer GEMM case; the tests call this too."""
    Mo, _, w = ONEPASS
    rng = np.random.default_rng(740)
    r = lambda s, n: o.bf16_round((s * rng.standard_normal((Mo, n))).astype(np.float32))
    return r(1e-3, w), np.concatenate([r(2.0, w), r(1.0, w)], axis=1)


def split3_inputs():
    """Three gradients [M, 512 | 256 | 256] of the three-split GEMM case; the tests call this too."""
    Mo = ONEPASS[0]
    rng = np.random.default_rng(760)
    return tuple(o.bf16_round((1e-3 * rng.standard_normal((Mo, w))).astype(np.float32)) for w in (512, 256, 256))


def rope_table(seq_len, pair_dim):
    """(cos, sin) fp32 [seq_len, pair_dim, 2] of seeded angles; the tests call this too."""
    ang = np.random.default_rng(790 + pair_dim).uniform(-np.pi, np.pi, size=(seq_len, pair_dim)).astype(np.float32)
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def inverse_rope_inputs():
    """dQ [256, 256], dK [256, 128], dV [256, 128] and a (cos, sin) table [128, 32, 2]; the tests call this too."""
    rng = np.random.default_rng(770)
    gs = tuple(o.bf16_round(rng.standard_normal((256, w)).astype(np.float32)) for w in (256, 128, 128))
    ang = rng.uniform(-np.pi, np.pi, size=(128, 32)).astype(np.float32)
    return gs, np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def load_reference_gemm_module():
    paths = glob.glob(os.path.join(ROOT, "oracle", "_ref", "_C_mx*.so"))
    if not paths:
        return None
    spec = importlib.util.spec_from_file_location("_C_mx", paths[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = load_reference_module()
    dev = torch.device("cuda", 0)
    out = {}
    for i, (name, fn, kind, extra) in enumerate(CASES):
        tensors = [torch.from_numpy(a).to(torch.bfloat16).to(dev) for a in make_inputs(kind, 300 + i)]
        r = getattr(ref, fn)(*tensors, *extra)
        torch.cuda.synchronize()
        for j, t in enumerate(r):
            if not torch.is_tensor(t):
                continue
            a = t.view(torch.uint8) if t.dtype not in (torch.float32, torch.uint8) else t
            out[f"{name}.{j}"] = a.cpu().numpy()
    ref_gemm = load_reference_gemm_module()
    if ref_gemm is not None:
        # quantised by the reference's quantiser (mode 1), multiplied by the reference's GEMM: D bf16, and D + R
        for i, shape in enumerate(GEMM_SHAPES):
            a, b = (torch.from_numpy(t).to(torch.bfloat16).to(dev) for t in gemm_operands(shape, 700 + i))
            qa, qb = ref.mxfp4_quantize_for_gemm(a, 1), ref.mxfp4_quantize_for_gemm(b, 1)
            d = torch.empty(shape[0], shape[1], dtype=torch.bfloat16, device=dev)
            ref_gemm.mxfp4_gemm(qa[0], qa[1], qb[0], qb[1], d)
            torch.cuda.synchronize()
            out[f"gemm_{i}.d"] = d.view(torch.int16).cpu().numpy()
            r = (0.5 * torch.randn(shape[0], shape[1], generator=torch.Generator().manual_seed(800 + i))).to(torch.bfloat16).to(dev)
            ref_gemm.mxfp4_gemm_residual(qa[0], qa[1], qb[0], qb[1], r, d)
            torch.cuda.synchronize()
            out[f"gemm_{i}.d_residual"] = d.view(torch.int16).cpu().numpy()
    if ref_gemm is not None:
        # the one-pass split2 dgrad (A = column concatenation of two row-quantised gradients, one weight per split,
        # all terms accumulated before the one rounding) and two batched products
        Mo, No, w = ONEPASS
        g1, g2 = (torch.from_numpy(gemm_operands((Mo, 1, w), 720 + i)[0] * 1e-3).to(torch.bfloat16).to(dev) for i in range(2))
        q1, q2 = ref.mxfp4_quantize_for_gemm(g1, 1), ref.mxfp4_quantize_for_gemm(g2, 1)
        a_full = torch.cat([q1[0].view(torch.uint8), q2[0].view(torch.uint8)], dim=1).contiguous()
        ws = [ref.mxfp4_quantize_for_gemm(torch.from_numpy(gemm_operands((1, No, w), 730 + i)[1]).to(torch.bfloat16).to(dev), 1)
              for i in range(2)]
        d = torch.empty(Mo, No, dtype=torch.bfloat16, device=dev)
        ref_gemm.mxfp4_split2_dgrad_strided_onepass_gemm(a_full.view(torch.float4_e2m1fn_x2), [q1[1], q2[1]], [0, w // 2], [w // 2, w // 2],
                                                         [ws[0][0], ws[1][0]], [ws[0][1], ws[1][1]], d, -1)
        torch.cuda.synchronize()
        out["onepass.d"] = d.view(torch.int16).cpu().numpy()
        d1, d2 = torch.empty_like(d), torch.empty_like(d)
        ref_gemm.mxfp4_batched_gemm([q1[0], q2[0]], [q1[1], q2[1]], [ws[0][0], ws[1][0]], [ws[0][1], ws[1][1]], [d1, d2])
        torch.cuda.synchronize()
        out["batched.0"], out["batched.1"] = d1.view(torch.int16).cpu().numpy(), d2.view(torch.int16).cpu().numpy()
    if ref_gemm is not None:
        # the reference's own call pattern (mxfp4_fused_linear.py:10390-10398, 10803-10829): the combined producer's
        # side-by-side row operand and column slices of its scale tensor into the one-pass split dgrad GEMM
        Mo, No, w = ONEPASS
        dh, h13 = combined_inputs()
        q = ref.mxfp4_fused_silu_deriv_quantize_split2_row_and_col_strided_combined(
            torch.from_numpy(dh).to(torch.bfloat16).to(dev), torch.from_numpy(h13).to(torch.bfloat16).to(dev), w, w, 1)
        ws = [ref.mxfp4_quantize_for_gemm(torch.from_numpy(gemm_operands((1, No, w), 730 + i)[1]).to(torch.bfloat16).to(dev), 1)
              for i in range(2)]
        d = torch.empty(Mo, No, dtype=torch.bfloat16, device=dev)
        ref_gemm.mxfp4_split2_dgrad_strided_onepass_gemm(q[0], [q[1].narrow(1, 0, w // 128), q[1].narrow(1, w // 128, w // 128)],
                                                         [0, w // 2], [w // 2, w // 2], [ws[0][0], ws[1][0]],
                                                         [ws[0][1], ws[1][1]], d, -1)
        torch.cuda.synchronize()
        out["onepass_combined.d"] = d.view(torch.int16).cpu().numpy()
    if ref_gemm is not None:
        # QKV dgrad as the reference runs it: split3 quantiser (no concatenation), then the three-split one-pass GEMM
        Mo, No, w = ONEPASS
        gs = split3_inputs()
        q = ref.mxfp4_quantize_split3_row_and_col(*(torch.from_numpy(t).to(torch.bfloat16).to(dev) for t in gs), 1)
        ws = [ref.mxfp4_quantize_for_gemm(torch.from_numpy(gemm_operands((1, No, t.shape[1]), 750 + i)[1]).to(torch.bfloat16).to(dev), 1)
              for i, t in enumerate(gs)]
        offs, a_scs, off = [], [], 0
        for t in gs:
            offs.append(off // 2)
            a_scs.append(q[1].narrow(1, off // 128, t.shape[1] // 128))
            off += t.shape[1]
        d = torch.empty(Mo, No, dtype=torch.bfloat16, device=dev)
        ref_gemm.mxfp4_split3_dgrad_strided_onepass_gemm(q[0], a_scs, offs, [t.shape[1] // 2 for t in gs], [x[0] for x in ws],
                                                         [x[1] for x in ws], d, -1)
        torch.cuda.synchronize()
        out["onepass_split3.d"] = d.view(torch.int16).cpu().numpy()
    if ref_gemm is not None:
        # GEMM with the rotary epilogue: heads of 64 (the 128-token table of the inverse-rotation case) and of 128
        for tag, shape, pair_dim in (("rope64", GEMM_SHAPES[0], 32), ("rope128", GEMM_SHAPES[1], 64)):
            a, b = (torch.from_numpy(t).to(torch.bfloat16).to(dev) for t in gemm_operands(shape, 780))
            qa, qb = ref.mxfp4_quantize_for_gemm(a, 1), ref.mxfp4_quantize_for_gemm(b, 1)
            cs = torch.from_numpy(rope_table(128, pair_dim)).to(dev)
            d = torch.empty(shape[0], shape[1], dtype=torch.bfloat16, device=dev)
            ref_gemm.mxfp4_gemm_rope_live64(qa[0], qa[1], qb[0], qb[1], d, cs, 128)
            torch.cuda.synchronize()
            out[f"gemm_{tag}.d"] = d.view(torch.int16).cpu().numpy()
            # the same rotation from separate cos / sin tables [seq_len, rotary_dim / 2]
            ref_gemm.mxfp4_gemm_rope(qa[0], qa[1], qb[0], qb[1], d, cs[..., 0].contiguous(), cs[..., 1].contiguous(), 128,
                                     2 * pair_dim, 2 * pair_dim)
            torch.cuda.synchronize()
            out[f"gemm_{tag}.d_tables"] = d.view(torch.int16).cpu().numpy()
    if ref_gemm is not None:
        # the fused QKV projection as the reference's backend calls it (mxfp4_backend.py:3153-3175): one activation,
        # three weights, Q and K with the rotary epilogue, V without (an empty table)
        shape = GEMM_SHAPES[0]
        a = torch.from_numpy(gemm_operands(shape, 781)[0]).to(torch.bfloat16).to(dev)
        qa = ref.mxfp4_quantize_for_gemm(a, 1)
        ws = [ref.mxfp4_quantize_for_gemm(torch.from_numpy(gemm_operands(shape, 782 + i)[1]).to(torch.bfloat16).to(dev), 1)
              for i in range(3)]
        cs = torch.from_numpy(rope_table(128, 32)).to(dev)
        ds = [torch.empty(shape[0], shape[1], dtype=torch.bfloat16, device=dev) for _ in range(3)]
        ref_gemm.mxfp4_batched_gemm_rope_live64([qa[0]] * 3, [qa[1]] * 3, [w[0] for w in ws], [w[1] for w in ws], ds,
                                                [cs, cs, torch.empty(0, dtype=torch.float32, device=dev)], [128, 128, 0])
        torch.cuda.synchronize()
        for i, d in enumerate(ds):
            out[f"batched_rope.{i}"] = d.view(torch.int16).cpu().numpy()
    # split3 with the inverse rotary embedding of the first two inputs folded in (sequence of 128 tokens, two per batch)
    gs, cs = inverse_rope_inputs()
    r = ref.mxfp4_quantize_split3_row_and_col_inverse_rope_live64(
        *(torch.from_numpy(t).to(torch.bfloat16).to(dev) for t in gs), torch.from_numpy(cs).to(dev), cs.shape[0], 1)
    torch.cuda.synchronize()
    for j, t in enumerate(r):
        out[f"split3_inverse_rope.{j}"] = (t.view(torch.uint8) if t.dtype != torch.uint8 else t).cpu().numpy()
    dst = os.environ.get("MX_GOLDEN_OUT", os.path.join(HERE, "mxfp4_reference_kernels_golden.npz"))
    np.savez_compressed(dst, **out)
    print(f"wrote {dst}: {len(out)} arrays, {os.path.getsize(dst)} bytes")


if __name__ == "__main__":
    main()
