"""Records outputs of further barrier-free kernels of the reference's OWN NVFP4 modules on seeded inputs.

Test infrastructure.  Needs one B200 and ``_tk_quant_v5`` + ``_C`` compiled by ``oracle/build_ref.sh <checkout> all`` into
``oracle/_ref/``.  Entry points (launch paths read in the reference: tensor-maximum kernel with a last-block counter,
ordinary element / tile kernels, the tuned TMA kernel, pipelined GEMM kernels — nothing spins on a grid-wide flag):

  _tk_quant_v5.tk_quantize_weight_2d                      16 x 16 weight tiles (tk_quantize.cu:2445-2555)
  _tk_quant_v5.tk_silu_mul_split_bf16 / tk_silu_deriv_split_bf16   the SwiGLU element kernels (:8923-8979)
  _tk_quant_v5.tk_group_quantize_dim1_split3_for_gemm     three gradient streams, SR on both axes = the two-pass route
                                                          of one tuned-kernel launch per stream (:6485-6548)
  _C.nvfp4_forward_rope_packed_qk / nvfp4_inverse_rope_packed_qk    (nvfp4_b200_gemm.cu:1183-1216)
  _C.nvfp4_grouped_gemm_rope_packed_split                 QKV projection with the rotary epilogue (:1406-1441)

    python tests/golden/make_misc_reference_golden.py     # writes tests/golden/nvfp4_misc_reference_golden.npz

Runs in ONE fresh process (the split3 case is first: its three stochastic launches take the numbers 0, 1, 2).
Inputs are regenerated from their seeds by the tests.
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

SEED, SUBSEQ = 20261127, 11
SPLIT3 = (256, (256, 128, 128))             # rows, widths of the three streams
ROPE = dict(M=256, seq=128, head=64, q_dim=512, kv_dim=256, K=512)


def grads(M, n, seed):
    return o.bf16_round((1e-3 * np.random.default_rng(seed).standard_normal((M, n))).astype(np.float32))


def normal(M, n, seed, s=1.0):
    return o.bf16_round((s * np.random.default_rng(seed).standard_normal((M, n))).astype(np.float32))


def rope_table(seq, head, seed):
    ang = np.random.default_rng(seed).uniform(0.0, 6.2831853, size=(seq, head // 2)).astype(np.float32)
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def _load(name):
    paths = glob.glob(os.path.join(ROOT, "oracle", "_ref", name + ".*.so"))
    if not paths:
        raise SystemExit(f"oracle/_ref/{name}*.so is missing: run oracle/build_ref.sh <reference checkout> all")
    spec = importlib.util.spec_from_file_location(name, paths[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    q, c = _load("_tk_quant_v5"), _load("_C")
    dev = torch.device("cuda", 0)
    t = lambda a: torch.from_numpy(a).to(torch.bfloat16).to(dev)
    u8 = lambda x: x.contiguous().view(torch.uint8).cpu().numpy()
    out = {}
    # split3, SR on both axes (first: launch numbers 0..2)
    M, widths = SPLIT3
    ins = [t(grads(M, n, 500 + i)) for i, n in enumerate(widths)]
    r = q.tk_group_quantize_dim1_split3_for_gemm(*ins, True, SEED, SUBSEQ, "both")
    torch.cuda.synchronize()
    out["split3.row_fp4_full"], out["split3.row_sc_cat"] = u8(r[5]), u8(r[6])
    out["split3.col_fp4_full"], out["split3.col_sc_cat"] = u8(r[7]), u8(r[8])
    out["split3.sg"], out["split3.amax"] = r[2].cpu().numpy(), r[12].cpu().numpy()
    # 16 x 16 weight tiles
    w = t(normal(256, 384, 510, 0.02))
    r = q.tk_quantize_weight_2d(w)
    torch.cuda.synchronize()
    for j in range(4):
        out[f"weight_2d.{j}"] = u8(r[j])
    out["weight_2d.sg"] = r[4].cpu().numpy()
    # SwiGLU element kernels
    h1, h3, dh = t(normal(256, 384, 520, 2.0)), t(normal(256, 384, 521)), t(grads(256, 384, 522))
    out["silu_mul"] = q.tk_silu_mul_split_bf16(h1, h3).view(torch.int16).cpu().numpy()
    d1, d3 = q.tk_silu_deriv_split_bf16(dh, h3, h1)
    torch.cuda.synchronize()
    out["silu_deriv.dh1"], out["silu_deriv.dh3"] = d1.view(torch.int16).cpu().numpy(), d3.view(torch.int16).cpu().numpy()
    # rotary embedding of packed Q / K and its inverse
    R = ROPE
    cs = torch.from_numpy(rope_table(R["seq"], R["head"], 530)).to(dev)
    qq, kk = t(normal(R["M"], R["q_dim"], 531)), t(normal(R["M"], R["kv_dim"], 532))
    qo, ko = torch.empty_like(qq), torch.empty_like(kk)
    c.nvfp4_forward_rope_packed_qk(qq, kk, cs, R["seq"], R["head"], qo, ko)
    torch.cuda.synchronize()
    out["rope_fwd.q"], out["rope_fwd.k"] = qo.view(torch.int16).cpu().numpy(), ko.view(torch.int16).cpu().numpy()
    c.nvfp4_inverse_rope_packed_qk(qq, kk, cs, R["seq"], R["head"], qo, ko)
    torch.cuda.synchronize()
    out["rope_inv.q"], out["rope_inv.k"] = qo.view(torch.int16).cpu().numpy(), ko.view(torch.int16).cpu().numpy()
    # QKV projection with the rotary epilogue.  The operands come from the reference's optional-mode quantiser with
    # data SR on (its round-to-nearest path runs a kernel with a grid-wide barrier) and are stored in the fixture, so
    # the test feeds the same packed operands to this library's GEMM.
    x = t(normal(R["M"], R["K"], 540))
    wq = t(normal(R["q_dim"] + 2 * R["kv_dim"], R["K"], 541, 0.02))
    qx = q.tk_quantize_for_gemm_opt(x, False, True, True, False, "none", False, SEED, SUBSEQ, 448.0, "row")
    qw = q.tk_quantize_for_gemm_opt(wq, False, True, True, False, "none", False, SEED, SUBSEQ, 448.0, "row")
    N = R["q_dim"] + 2 * R["kv_dim"]
    b_sg = qw[4].expand(N // 256).contiguous()
    dq = torch.empty(R["M"], R["q_dim"], dtype=torch.bfloat16, device=dev)
    dk = torch.empty(R["M"], R["kv_dim"], dtype=torch.bfloat16, device=dev)
    dv = torch.empty(R["M"], R["kv_dim"], dtype=torch.bfloat16, device=dev)
    c.nvfp4_grouped_gemm_rope_packed_split(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, cs, R["seq"], R["head"], R["head"])
    torch.cuda.synchronize()
    out["qkv_rope.a_fp4"], out["qkv_rope.a_sc"], out["qkv_rope.a_sg"] = u8(qx[0]), u8(qx[1]), qx[4].cpu().numpy()
    out["qkv_rope.b_fp4"], out["qkv_rope.b_sc"], out["qkv_rope.b_sg"] = u8(qw[0]), u8(qw[1]), qw[4].cpu().numpy()
    for name, d in (("q", dq), ("k", dk), ("v", dv)):
        out[f"qkv_rope.{name}"] = d.view(torch.int16).cpu().numpy()
    dst = os.environ.get("MISC_GOLDEN_OUT", os.path.join(HERE, "nvfp4_misc_reference_golden.npz"))
    np.savez_compressed(dst, **out)
    print(f"wrote {dst}: {len(out)} arrays, {os.path.getsize(dst)} bytes")


if __name__ == "__main__":
    main()
