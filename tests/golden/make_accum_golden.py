"""Records the output bytes of the reference's OWN nvfp4_batched_accum_gemm kernel on seeded operands.

Test infrastructure.  Needs one B200 and the reference's ``_C`` extension module compiled by ``oracle/build_ref.sh``
into ``oracle/_ref/`` (the reference's sources are not needed at run time):

    python tests/golden/make_accum_golden.py        # writes tests/golden/nvfp4_accum_reference_golden.npz

The kernel (nvfp4_batched_accum_gemm.cuh) is an ordinary pipelined GEMM kernel: its waits are on shared-memory
barriers of its own cluster, it has no grid-wide software barrier.  The operands are quantised by this library from
inputs the test regenerates from their seeds (make_terms below), so the fixture holds the reference's outputs only
(a SHA-256 of every output matrix and every eighth row of it): what they pin is the order in which the terms' scaled accumulators are added in fp32.
"""
import glob
import hashlib
import importlib
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import fp4_oracle as o  # noqa: E402

M, N, K = 512, 512, 512     # four 256 x 256 tiles (the reference's launch needs more than one)


def make_terms(n):
    """Quantised operand pairs (A_i [M, K], B_i [N, K]) of n terms; the tests call this too."""
    tkq = importlib.import_module("mfu-fp4-training_b200.tk_quant_v5")
    terms = []
    for i in range(n):
        x = o.make_activations(M, K, seed=700 + i)
        w = o.bf16_round((0.02 * np.random.default_rng(800 + i).standard_normal((N, K))).astype(np.float32))
        qx = tkq.tk_quantize_for_gemm(torch.from_numpy(x).to(torch.bfloat16).cuda(), False, True)
        qw = tkq.tk_quantize_for_gemm(torch.from_numpy(w).to(torch.bfloat16).cuda(), False, True)
        terms.append((qx, qw))
    return terms


def split(terms):
    return ([t[0][0] for t in terms], [t[0][1] for t in terms], [t[0][4] for t in terms],
            [t[1][0] for t in terms], [t[1][1] for t in terms], [t[1][4] for t in terms])


def main():
    paths = glob.glob(os.path.join(ROOT, "oracle", "_ref", "_C*.so"))
    if not paths:
        raise SystemExit("oracle/_ref/_C*.so is missing: run oracle/build_ref.sh <reference checkout> gemm")
    spec = importlib.util.spec_from_file_location("_C", paths[0])
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {}
    terms = make_terms(4)
    for n in (2, 3, 4):
        d = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        ref.nvfp4_batched_accum_gemm(*split(terms[:n]), d)
        torch.cuda.synchronize()
        bits = d.view(torch.int16).cpu().numpy()
        out[f"sha256_{n}"] = np.frombuffer(hashlib.sha256(bits.tobytes()).digest(), dtype=np.uint8)   # of all M x N outputs
        out[f"rows_{n}"] = bits[::8].copy()                                                          # every eighth row, to locate a difference
    dst = os.environ.get("ACCUM_GOLDEN_OUT", os.path.join(HERE, "nvfp4_accum_reference_golden.npz"))
    np.savez_compressed(dst, **out)
    print(f"wrote {dst}: {os.path.getsize(dst)} bytes")


if __name__ == "__main__":
    main()
