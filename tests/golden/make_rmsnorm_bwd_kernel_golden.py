"""Records the outputs of the reference's OWN RMSNorm-backward kernels (`_C.sum3_rmsnorm_bwd_out`,
`_C.rmsnorm_bwd_residual_out`, nvfp4_b200_gemm.cu:300-646) on seeded inputs.

Test infrastructure.  Needs one B200 and the reference's ``_C`` module compiled by ``oracle/build_ref.sh <checkout>
gemm`` into ``oracle/_ref/``.  The kernels are ordinary launches (one CTA per row for dx, fixed 256-row tiles and a
reduction launch for dgamma; the residual form adds its dgamma with atomics): nothing waits on another CTA.

    python tests/golden/make_rmsnorm_bwd_kernel_golden.py   # writes tests/golden/rmsnorm_bwd_kernels_golden.npz

Inputs are regenerated from their seeds by the tests (``make_inputs``); the fixture holds inv_rms and the outputs.
Matrices are stored as the SHA-256 of all their bytes plus every eighth row (``pack``), small vectors whole.
"""
import hashlib
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

SUM3_SHAPES = [(256, 512), (300, 4096), (768, 1024)]   # 300 rows: a partial last dgamma tile
RESIDUAL_ROWS = [256, 300]
EPS = 1e-5


def make_inputs(M, K, seed):
    """(d0, d1, d2, x, gamma) as float32 arrays of bf16 values."""
    rng = np.random.default_rng(seed)
    d = [o.bf16_round((1e-3 * rng.standard_normal((M, K))).astype(np.float32)) for _ in range(3)]
    return (*d, o.make_activations(M, K, seed=seed + 1), o.make_gamma(K, seed=seed + 2))


def pack(out, key, array):
    """sha256 of the whole array + every eighth row of it."""
    a = np.ascontiguousarray(array)
    out[key + ".sha256"] = np.frombuffer(hashlib.sha256(a.tobytes()).digest(), dtype=np.uint8)
    out[key + ".rows8"] = a[::8].copy()


def main():
    paths = glob.glob(os.path.join(ROOT, "oracle", "_ref", "_C.*.so"))
    if not paths:
        raise SystemExit("oracle/_ref/_C*.so is missing: run oracle/build_ref.sh <reference checkout> gemm")
    spec = importlib.util.spec_from_file_location("_C", paths[0])
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    dev = torch.device("cuda", 0)
    bits = lambda t: t.view(torch.int16).cpu().numpy()
    out = {}
    for i, (M, K) in enumerate(SUM3_SHAPES):
        d0, d1, d2, x, gamma = (torch.from_numpy(a).to(torch.bfloat16).to(dev) for a in make_inputs(M, K, 900 + i))
        inv = torch.rsqrt(x.float().pow(2).mean(dim=1) + EPS).contiguous()
        d_sum, dx = torch.empty_like(x), torch.empty_like(x)
        partials = torch.zeros((M + 255) // 256, K, dtype=torch.float32, device=dev)
        dgamma = torch.zeros(K, dtype=torch.float32, device=dev)
        ref.sum3_rmsnorm_bwd_out(d0, d1, d2, x, gamma, inv, d_sum, dx, partials, dgamma)
        torch.cuda.synchronize()
        out[f"sum3_{i}.inv_rms"] = inv.cpu().numpy()
        pack(out, f"sum3_{i}.d_sum", bits(d_sum))
        pack(out, f"sum3_{i}.dx", bits(dx))
        out[f"sum3_{i}.partials"], out[f"sum3_{i}.dgamma"] = partials.cpu().numpy(), dgamma.cpu().numpy()
    for i, M in enumerate(RESIDUAL_ROWS):
        K = 4096
        d0, d1, _, x, gamma = (torch.from_numpy(a).to(torch.bfloat16).to(dev) for a in make_inputs(M, K, 950 + i))
        inv = torch.rsqrt(x.float().pow(2).mean(dim=1) + EPS).contiguous()
        dx = torch.empty_like(x)
        dgamma = torch.zeros(K, dtype=torch.float32, device=dev)
        ref.rmsnorm_bwd_residual_out(d0, x, gamma, inv, d1, dx, dgamma)
        torch.cuda.synchronize()
        out[f"residual_{i}.inv_rms"] = inv.cpu().numpy()
        pack(out, f"residual_{i}.dx", bits(dx))
        out[f"residual_{i}.dgamma"] = dgamma.cpu().numpy()
    dst = os.environ.get("RMS_BWD_GOLDEN_OUT", os.path.join(HERE, "rmsnorm_bwd_kernels_golden.npz"))
    np.savez_compressed(dst, **out)
    print(f"wrote {dst}: {len(out)} arrays, {os.path.getsize(dst)} bytes")


if __name__ == "__main__":
    main()
