"""Records the output bytes of the reference's OWN sm_100a quantiser kernels on seeded inputs.

Test infrastructure.  Needs one B200 and the reference's ``_tk_quant_v5`` extension module compiled by
``oracle/build_ref.sh`` into ``oracle/_ref/`` (the reference's sources are not needed at run time):

    python tests/golden/make_sr_golden.py            # writes tests/golden/nvfp4_sr_reference_golden.npz

Only entry points whose launch path has no grid-wide software barrier are called (read in the reference's
tk_quantize.cu): ``tk_quantize_for_gemm_opt`` with at least one optional mode on (tensor-maximum kernel with a
last-block counter, Hadamard scans, the tuned TMA kernel ``quantize_transpose_tuned.cuh``; with every mode off it
would fall through to the persistent kernels, :4369-4375) and ``tk_fused_norm_quantize`` in its default,
barrier-free branch (:8048-8108).  ``USE_TK_NORM_QUANT_TWO_PASS`` must not be set to 0.

Inputs are regenerated from their seeds by the tests (oracle.make_activations / make_gamma / make_gradient), so the
fixture holds outputs only.  Calls run in the order of CASES in ONE fresh process: the reference numbers its
stochastic launches with a device-side counter that starts at 0 (tk_quantize.cu:443-481), and the fixture records
how many launches each case consumed.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import fp4_oracle as o  # noqa: E402

SEED, SUBSEQ = 20261125, 7

# name -> (shape, input kind, kwargs of tk_quantize_for_gemm_opt)
CASES = [
    ("sr_both_dc", (256, 384), "grad", dict(return_transpose=True, encode_centric=False, data_sr=True, scale_sr=False, rht="none", sign=False, sr_axes="both")),
    ("sr_row_dc", (256, 384), "grad", dict(return_transpose=True, encode_centric=False, data_sr=True, scale_sr=False, rht="none", sign=False, sr_axes="row")),
    ("sr_col_dc", (256, 384), "grad", dict(return_transpose=True, encode_centric=False, data_sr=True, scale_sr=False, rht="none", sign=False, sr_axes="col")),
    ("sr_both_ec", (128, 256), "act", dict(return_transpose=True, encode_centric=True, data_sr=True, scale_sr=False, rht="none", sign=False, sr_axes="both")),
    ("sr_scale_dc", (256, 384), "grad", dict(return_transpose=True, encode_centric=False, data_sr=True, scale_sr=True, rht="none", sign=False, sr_axes="both")),
    ("scale_only_ec", (128, 256), "act", dict(return_transpose=True, encode_centric=True, data_sr=False, scale_sr=True, rht="none", sign=False, sr_axes="both")),
    ("scale_only_ec_zero_blocks", (128, 256), "act_zero", dict(return_transpose=True, encode_centric=True, data_sr=False, scale_sr=True, rht="none", sign=False, sr_axes="both")),
    ("sr_scale_ec_zero_blocks", (128, 256), "act_zero", dict(return_transpose=True, encode_centric=True, data_sr=True, scale_sr=True, rht="none", sign=False, sr_axes="both")),
    ("rht_row", (256, 384), "act", dict(return_transpose=True, encode_centric=False, data_sr=False, scale_sr=False, rht="row", sign=False, sr_axes="both")),
    ("rht_col", (256, 384), "act", dict(return_transpose=True, encode_centric=False, data_sr=False, scale_sr=False, rht="col", sign=False, sr_axes="both")),
    ("rht_both", (256, 384), "act", dict(return_transpose=True, encode_centric=False, data_sr=False, scale_sr=False, rht="both", sign=False, sr_axes="both")),
    ("rht_col_sr_col", (256, 384), "grad", dict(return_transpose=True, encode_centric=False, data_sr=True, scale_sr=False, rht="col", sign=False, sr_axes="col")),
    ("rht_col_sign", (256, 384), "act", dict(return_transpose=True, encode_centric=False, data_sr=False, scale_sr=False, rht="col", sign=True, sr_axes="both")),
    ("rht_both_sign_sr", (256, 384), "grad", dict(return_transpose=True, encode_centric=False, data_sr=True, scale_sr=False, rht="both", sign=True, sr_axes="both")),
    ("sr_row_only_no_transpose", (256, 384), "grad", dict(return_transpose=False, encode_centric=False, data_sr=True, scale_sr=False, rht="none", sign=False, sr_axes="row")),
    ("target_256", (128, 256), "act", dict(return_transpose=True, encode_centric=False, data_sr=True, scale_sr=False, rht="none", sign=False, sr_axes="both", target=256.0)),
]


def make_input(kind, shape, seed):
    """The seeded inputs of the cases; the tests call this too."""
    M, K = shape
    if kind == "grad":
        return o.bf16_round((1e-3 * np.random.default_rng(seed).standard_normal((M, K))).astype(np.float32))
    x = o.make_activations(M, K, seed=seed)
    if kind == "act_zero":   # all-zero 16-blocks in both orientations: a 32 x 32 corner and two scattered row blocks
        x = x.copy()
        x[:32, :32] = 0.0
        x[77, 64:80] = 0.0
        x[100, 240:256] = 0.0
    return x


def load_reference_module():
    import glob
    paths = glob.glob(os.path.join(ROOT, "oracle", "_ref", "_tk_quant_v5*.so"))
    if not paths:
        raise SystemExit("oracle/_ref/_tk_quant_v5*.so is missing: run oracle/build_ref.sh <reference checkout> quant")
    spec = importlib.util.spec_from_file_location("_tk_quant_v5", paths[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    if os.environ.get("USE_TK_NORM_QUANT_TWO_PASS", "1") in ("0", "false", "FALSE", "off"):
        raise SystemExit("USE_TK_NORM_QUANT_TWO_PASS=0 selects a kernel with a grid-wide software barrier: not run")
    ref = load_reference_module()
    dev = torch.device("cuda", 0)
    out = {}
    launches = 0
    for i, (name, shape, kind, kw) in enumerate(CASES):
        x = torch.from_numpy(make_input(kind, shape, 100 + i)).to(torch.bfloat16).to(dev)
        r = ref.tk_quantize_for_gemm_opt(x, kw["return_transpose"], kw["encode_centric"], kw["data_sr"], kw["scale_sr"], kw["rht"],
                                         kw["sign"], SEED, SUBSEQ, kw.get("target", 448.0), kw["sr_axes"])
        torch.cuda.synchronize()
        uses_sr = kw["data_sr"] or kw["scale_sr"]
        # one tuned-kernel launch when both operands round alike, else one per operand (tk_quantize.cu:4418-4520)
        row_sr = kw["data_sr"] and kw["sr_axes"] in ("row", "both")
        col_sr = kw["data_sr"] and kw["sr_axes"] in ("col", "both")
        # one tuned-kernel launch when both operands round alike and are quantised from the input itself, else one
        # per operand; every launch of a stochastic call takes a number (tk_quantize.cu:4375-4520)
        has_row_rht, has_col_rht = kw["rht"] in ("row", "both"), kw["rht"] in ("col", "both")
        rotated_copy = kw["sign"] and (has_row_rht or has_col_rht)   # the sign mask disables the in-kernel transform
        n = 0
        if uses_sr:
            n = 1 if (not kw["return_transpose"] or (row_sr == col_sr and not rotated_copy)) else 2
        out[f"{name}.first_launch"] = np.int64(launches)
        out[f"{name}.launches"] = np.int64(n)
        launches += n
        out[f"{name}.row_fp4"] = r[0].view(torch.uint8).cpu().numpy()
        out[f"{name}.row_sc"] = r[1].view(torch.uint8).cpu().numpy().reshape(-1)
        if kw["return_transpose"]:
            out[f"{name}.col_fp4"] = r[2].view(torch.uint8).cpu().numpy()
            out[f"{name}.col_sc"] = r[3].view(torch.uint8).cpu().numpy().reshape(-1)
        out[f"{name}.sg_row"] = r[4].cpu().numpy()
        out[f"{name}.sg_col"] = r[5].cpu().numpy()
    # fused RMSNorm + quantisation, round to nearest, encode-centric: the default barrier-free producer
    for tag, shape in (("norm_256x384", (256, 384)), ("norm_512x1024", (512, 1024))):
        M, K = shape
        x = torch.from_numpy(o.make_activations(M, K, seed=M + K)).to(torch.bfloat16).to(dev)
        gamma = torch.from_numpy(o.make_gamma(K, seed=K)).to(torch.bfloat16).to(dev)
        r = ref.tk_fused_norm_quantize(x, gamma, 1e-5, False, True)
        torch.cuda.synchronize()
        out[f"{tag}.row_fp4"] = r[0].view(torch.uint8).cpu().numpy()
        out[f"{tag}.row_sc"] = r[1].view(torch.uint8).cpu().numpy().reshape(-1)
        out[f"{tag}.col_fp4"] = r[2].view(torch.uint8).cpu().numpy()
        out[f"{tag}.col_sc"] = r[3].view(torch.uint8).cpu().numpy().reshape(-1)
        out[f"{tag}.sg"] = r[4].cpu().numpy()
        out[f"{tag}.inv_rms"] = r[5].cpu().numpy()
        out[f"{tag}.amax"] = r[6].cpu().numpy()
    dst = os.environ.get("SR_GOLDEN_OUT", os.path.join(HERE, "nvfp4_sr_reference_golden.npz"))
    np.savez_compressed(dst, **out)
    print(f"wrote {dst}: {len(out)} arrays, {launches} stochastic launches, {os.path.getsize(dst)} bytes")


if __name__ == "__main__":
    main()
