"""The CPU oracle against bytes the reference's OWN compiled kernels produced (fixtures recorded on a B200 by the
make_*_reference_golden.py scripts beside them): the oracle, not only the CUDA path, is pinned by the reference itself
for the round-to-nearest tuned kernel, the MXFP4 quantisers, both weight-tile forms, the rotary embedding and the RMSNorm
backward.  No GPU needed."""
import hashlib
import os

import numpy as np
import pytest

from oracle import fp4_oracle as o

GOLD_DIR = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    path = os.path.join(GOLD_DIR, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} not recorded")
    return np.load(path)


def _flat_eq(got, want):
    got, want = np.asarray(got).reshape(-1), np.asarray(want).reshape(-1)
    return got.size == want.size and bool((got == want).all())


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_mxfp4_row_and_col_quantiser(mode):
    from tests.golden import make_mx_reference_golden as G
    gold = _load("mxfp4_reference_kernels_golden.npz")
    (x,) = G.make_inputs("x", 300 + mode)
    ref = o.mxfp4_quantize_row_and_col(x, mode)
    for j, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
        assert _flat_eq(ref[k], gold[f"rowcol_m{mode}.{j}"]), k


def test_mxfp4_weight_tiles():
    from tests.golden import make_mx_reference_golden as G
    gold = _load("mxfp4_reference_kernels_golden.npz")
    (w,) = G.make_inputs("w", 304)
    ref = o.mxfp4_quantize_weight_2d(w)
    keys = ["row_fp4", "row_sc", "col_fp4", "col_sc"]
    got = [ref[k] for k in keys] if isinstance(ref, dict) else list(ref)
    for j in range(4):
        assert _flat_eq(got[j], gold[f"weight_2d.{j}"]), keys[j]


def test_nvfp4_weight_tiles():
    from tests.golden import make_misc_reference_golden as G
    gold = _load("nvfp4_misc_reference_golden.npz")
    w = G.normal(256, 384, 510, 0.02)
    amax = o.tensor_amax(w)
    row_fp4, row_sc, col_fp4, col_sc = o.nvfp4_quantize_2d(w, amax)
    assert _flat_eq(row_fp4, gold["weight_2d.0"]) and _flat_eq(col_fp4, gold["weight_2d.2"])
    assert _flat_eq(o.swizzle_scales(row_sc), gold["weight_2d.1"]) and _flat_eq(o.swizzle_scales(col_sc), gold["weight_2d.3"])
    assert np.float32(o.nvfp4_global_decode_scale(amax)) == gold["weight_2d.sg"].reshape(-1)[0]


@pytest.mark.parametrize("idx", [0, 1, 2, 3, 4, 5])
def test_tuned_kernel_round_to_nearest_and_hadamard_forms(idx):
    from tests.golden import make_opt_more_reference_golden as G
    gold = _load("nvfp4_opt_more_reference_golden.npz")
    name, sr, ec, ssr, rr, cr, rt, ret_row = G.TRANSPOSE_CASES[idx]
    assert not sr and not ssr
    x = G.transpose_input(idx)
    amax = o.tensor_amax(x)
    ref = o.nvfp4_quantize_transpose_launch(x, amax, amax, rt, False, ec, rr, cr, ret_row)
    if ret_row:
        assert _flat_eq(ref["row_fp4"], gold[f"{name}.0"]) and _flat_eq(ref["row_sc"], gold[f"{name}.1"])
    if rt:
        assert _flat_eq(ref["col_fp4"], gold[f"{name}.2"]) and _flat_eq(ref["col_sc"], gold[f"{name}.3"])


def test_rotary_embedding_of_packed_q_k():
    from tests.golden import make_misc_reference_golden as G
    gold = _load("nvfp4_misc_reference_golden.npz")
    R = G.ROPE
    cs = G.rope_table(R["seq"], R["head"], 530)
    q, k = G.normal(R["M"], R["q_dim"], 531), G.normal(R["M"], R["kv_dim"], 532)
    for tag, inverse in (("rope_fwd", False), ("rope_inv", True)):
        assert _flat_eq(o.bf16_bits(o.rope_packed(q, cs, inverse)).astype(np.int16), gold[f"{tag}.q"])
        assert _flat_eq(o.bf16_bits(o.rope_packed(k, cs, inverse)).astype(np.int16), gold[f"{tag}.k"])


@pytest.mark.parametrize("idx", [0, 2])
def test_rmsnorm_backward_three_stream_form(idx):
    from tests.golden import make_rmsnorm_bwd_kernel_golden as G
    gold = _load("rmsnorm_bwd_kernels_golden.npz")
    M, K = G.SUM3_SHAPES[idx]
    d0, d1, d2, x, gamma = G.make_inputs(M, K, 900 + idx)
    inv = gold[f"sum3_{idx}.inv_rms"]
    ref = o.sum3_rmsnorm_bwd(d0, d1, d2, x, gamma, inv)
    d_sum, dx, partials, dgamma = (ref[k] for k in ("d_sum", "grad_input", "dgamma_partials", "dgamma"))
    for key, arr in (("d_sum", d_sum), ("dx", dx)):
        bits = np.ascontiguousarray(o.bf16_bits(arr).astype(np.int16))
        assert _flat_eq(bits[::8], gold[f"sum3_{idx}.{key}.rows8"]), key
        digest = np.frombuffer(hashlib.sha256(bits.tobytes()).digest(), dtype=np.uint8)
        assert _flat_eq(digest, gold[f"sum3_{idx}.{key}.sha256"]), key
    assert _flat_eq(np.asarray(partials, dtype=np.float32), gold[f"sum3_{idx}.partials"])
    assert _flat_eq(np.asarray(dgamma, dtype=np.float32), gold[f"sum3_{idx}.dgamma"])


def test_rmsnorm_backward_residual_form():
    from tests.golden import make_rmsnorm_bwd_kernel_golden as G
    gold = _load("rmsnorm_bwd_kernels_golden.npz")
    M, K = G.RESIDUAL_ROWS[0], 4096
    d0, d1, _, x, gamma = G.make_inputs(M, K, 950)
    ref = o.rmsnorm_bwd_residual(d0, x, gamma, gold["residual_0.inv_rms"], d1)
    bits = np.ascontiguousarray(o.bf16_bits(ref["grad_input"]).astype(np.int16))
    assert _flat_eq(bits[::8], gold["residual_0.dx.rows8"])
    assert _flat_eq(np.frombuffer(hashlib.sha256(bits.tobytes()).digest(), dtype=np.uint8), gold["residual_0.dx.sha256"])
    want = gold["residual_0.dgamma"]
    assert np.abs(ref["dgamma"] - want).max() <= 1e-5 * np.abs(want).max()
