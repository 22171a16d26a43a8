"""GPU parity against bytes the reference's OWN sm_100a kernels produced (tests/golden/nvfp4_sr_reference_golden.npz,
recorded by tests/golden/make_sr_golden.py from the reference's compiled ``_tk_quant_v5`` module on a B200):
``tk_quantize_for_gemm_opt`` with Philox stochastic rounding of codes and of scale bytes, the 16-point Hadamard
transform on either axis, the sign mask, a non-default tensor-scale target, and the fused RMSNorm producer.  This
pins what a restatement from source cannot: which random word the reference's thread gives to which element, the
sign hash, the launch numbering, the scan that feeds each orientation's tensor scale.  Bit-exact, no tolerance."""
import os

import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.golden import make_sr_golden as G
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16, u8

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "nvfp4_sr_reference_golden.npz"))


@pytest.mark.parametrize("idx", range(len(G.CASES)), ids=[c[0] for c in G.CASES])
def test_opt_quantiser_reproduces_the_reference_kernels_bytes(idx):
    name, shape, kind, kw = G.CASES[idx]
    tkq = mod("tk_quant_v5")
    x = to_dev_bf16(G.make_input(kind, shape, 100 + idx))
    first = int(GOLD[f"{name}.first_launch"])
    tkq.tk_set_sr_invocation_count(first)       # the reference numbered its launches from a fresh process
    r = tkq.tk_quantize_for_gemm_opt(x, kw["return_transpose"], kw["encode_centric"], kw["data_sr"], kw["scale_sr"], kw["rht"],
                                     kw["sign"], G.SEED, G.SUBSEQ, kw.get("target", 448.0), kw["sr_axes"])
    torch.cuda.synchronize()
    assert tkq.tk_sr_invocation_count() - first == int(GOLD[f"{name}.launches"])
    keys = [("row_fp4", 0), ("row_sc", 1)] + ([("col_fp4", 2), ("col_sc", 3)] if kw["return_transpose"] else [])
    for k, i in keys:
        got, want = u8(r[i]).reshape(-1), GOLD[f"{name}.{k}"].reshape(-1)
        assert np.array_equal(got, want), f"{name}.{k}: {(got != want).sum()} of {got.size} bytes differ from the reference kernel's"
    assert r[4].item() == GOLD[f"{name}.sg_row"][0] and r[5].item() == GOLD[f"{name}.sg_col"][0]
    assert_status_ok()


@pytest.mark.parametrize("tag,shape", [("norm_256x384", (256, 384)), ("norm_512x1024", (512, 1024))])
def test_fused_rmsnorm_producer_reproduces_the_reference_kernels_bytes(tag, shape):
    """tk_fused_norm_quantize (round to nearest, encode-centric, row + column operands): codes, scale bytes, tensor
    scale and the per-row inverse RMS, all bit for bit."""
    tkq = mod("tk_quant_v5")
    M, K = shape
    x = to_dev_bf16(o.make_activations(M, K, seed=M + K))
    gamma = to_dev_bf16(o.make_gamma(K, seed=K))
    r = tkq.tk_fused_norm_quantize(x, gamma, 1e-5, False, True)
    torch.cuda.synchronize()
    for k, i in (("row_fp4", 0), ("row_sc", 1), ("col_fp4", 2), ("col_sc", 3)):
        got, want = u8(r[i]).reshape(-1), GOLD[f"{tag}.{k}"].reshape(-1)
        assert np.array_equal(got, want), f"{tag}.{k}: {(got != want).sum()} of {got.size} bytes differ"
    assert r[4].item() == GOLD[f"{tag}.sg"][0]
    assert np.array_equal(r[5].cpu().numpy(), GOLD[f"{tag}.inv_rms"])
    assert r[6].item() == GOLD[f"{tag}.amax"][0]
    assert_status_ok()
