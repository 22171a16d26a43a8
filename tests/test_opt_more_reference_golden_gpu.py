"""GPU parity against outputs of three more entry points of the reference's OWN compiled ``_tk_quant_v5`` module
(tests/golden/nvfp4_opt_more_reference_golden.npz, recorded by tests/golden/make_opt_more_reference_golden.py on a
B200): `tk_quantize_transpose` (the tuned kernel with given tensor maxima: round to nearest under both scale rules,
one operand switched off, Hadamard forms, stochastic codes and scale bytes), `tk_fused_norm_quantize_opt` with
stochastic rounding, and `tk_silu_deriv_quantize_split_for_gemm_opt` in five rounding modes.  Bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.golden import make_opt_more_reference_golden as G
from tests.golden.make_misc_reference_golden import grads, normal
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16

pytestmark = pytest.mark.gpu

_PATH = os.path.join(os.path.dirname(__file__), "golden", "nvfp4_opt_more_reference_golden.npz")
GOLD = np.load(_PATH) if os.path.exists(_PATH) else None
needs_fixture = pytest.mark.skipif(GOLD is None, reason="fixture not recorded")
_u8 = lambda t: t.contiguous().view(torch.uint8).cpu().numpy()


def _eq(key, got):
    want = GOLD[key]
    assert got.size == want.size, key
    bad = int((got.reshape(-1) != want.reshape(-1)).sum())
    assert bad == 0, f"{key}: {bad} of {got.size} values differ from the reference kernel's"


def _launches_before(kind, idx):
    """Stochastic launches the reference's fresh process had numbered before this case (the generator's order)."""
    n = 0                                                     # tk_quantize_transpose takes its state from the caller
    cases = [("norm", c) for c in G.NORM_CASES] + [("split2", c) for c in G.SPLIT2_CASES]
    for k, c in cases:
        if k == kind and c is (G.NORM_CASES if kind == "norm" else G.SPLIT2_CASES)[idx]:
            return n
        if k == "norm":
            n += 1 if (c[2] or c[3]) else 0
        else:
            sr, ssr = c[2], c[3]
            n += 2 if (sr or ssr) else 0                      # one number per tensor of the pair (dh1, dh3)
    return n


@needs_fixture
@pytest.mark.parametrize("idx", range(len(G.TRANSPOSE_CASES)), ids=[c[0] for c in G.TRANSPOSE_CASES])
def test_quantize_transpose(idx):
    name, sr, ec, ssr, rr, cr, rt, ret_row = G.TRANSPOSE_CASES[idx]
    tkq = mod("tk_quant_v5")
    x = to_dev_bf16(G.transpose_input(idx))
    amax = x.float().abs().max().reshape(1).contiguous()
    state = torch.tensor([G.SEED, G.SUBSEQ + (idx << 32)], dtype=torch.int64, device="cuda")
    r = tkq.tk_quantize_transpose(x, amax, amax, rt, sr, ec, ssr, rr, cr, ret_row, state)
    torch.cuda.synchronize()
    M, K = G.SHAPE
    want_shapes = [(M, K // 2), (M, K // 16), (K, M // 2), (K, M // 16)]
    for j in range(4):
        key = f"{name}.{j}"
        if key in GOLD.files:
            assert tuple(r[j].shape) == want_shapes[j] and r[j].dtype == torch.uint8
            if j >= 2 or ret_row:          # with return_row off the row tensors are returned unwritten, by both
                _eq(key, _u8(r[j]))
        else:
            assert r[j].numel() == 0
    assert_status_ok()


@needs_fixture
@pytest.mark.parametrize("idx", range(len(G.NORM_CASES)), ids=[c[0] for c in G.NORM_CASES])
def test_fused_norm_quantize_opt(idx):
    name, ec, sr, ssr = G.NORM_CASES[idx]
    tkq = mod("tk_quant_v5")
    M, K = G.SHAPE
    x, g = to_dev_bf16(o.make_activations(M, K, seed=1100 + idx)), to_dev_bf16(o.make_gamma(K, seed=1110 + idx))
    tkq.tk_set_sr_invocation_count(_launches_before("norm", idx))
    r = tkq.tk_fused_norm_quantize_opt(x, g, 1e-5, True, ec, sr, ssr, "row", False, G.SEED, G.SUBSEQ)
    torch.cuda.synchronize()
    for j in range(4):
        _eq(f"{name}.{j}", _u8(r[j]))
    assert r[4].item() == GOLD[f"{name}.sg_row"].reshape(-1)[0] and r[5].item() == GOLD[f"{name}.sg_col"].reshape(-1)[0]
    assert np.array_equal(r[6].cpu().numpy(), GOLD[f"{name}.inv_rms"])
    assert_status_ok()


@needs_fixture
@pytest.mark.parametrize("idx", range(len(G.SPLIT2_CASES)), ids=[c[0] for c in G.SPLIT2_CASES])
def test_silu_deriv_quantize_split_opt(idx):
    name, ec, sr, ssr, rht, axes = G.SPLIT2_CASES[idx]
    tkq = mod("tk_quant_v5")
    M, K = G.SHAPE
    dh, h3, h1 = to_dev_bf16(grads(M, K, 1200 + idx)), to_dev_bf16(normal(M, K, 1210 + idx)), to_dev_bf16(normal(M, K, 1220 + idx, 2.0))
    tkq.tk_set_sr_invocation_count(_launches_before("split2", idx))
    r = tkq.tk_silu_deriv_quantize_split_for_gemm_opt(dh, h3, h1, True, ec, sr, ssr, rht, False, G.SEED, G.SUBSEQ, axes)
    torch.cuda.synchronize()
    _eq(f"{name}.dh1", r[13].view(torch.int16).cpu().numpy())
    _eq(f"{name}.dh3", r[14].view(torch.int16).cpu().numpy())
    for j in (4, 5, 10, 11, 12):
        assert np.array_equal(r[j].cpu().numpy().reshape(-1), GOLD[f"{name}.{j}"].reshape(-1)), f"{name}.{j}"
    for j in (0, 1, 2, 3, 6, 7, 8, 9):
        _eq(f"{name}.{j}", _u8(r[j]))
    assert_status_ok()
