"""GPU parity against bytes the reference's OWN sm_100a MXFP4 kernels produced
(tests/golden/mxfp4_reference_kernels_golden.npz, recorded by tests/golden/make_mx_reference_golden.py from the
reference's compiled ``mxfp4_quant_v4`` module on a B200): round-to-nearest row / column quantisers in the three
exponent modes, the 32 x 32 weight form, the fused RMSNorm, SwiGLU and SiLU-derivative producers (whose element
arithmetic — ``__expf``, the division — is the reference kernel's, not a CPU restatement's), and the stochastic /
Hadamard forms with their Philox streams and launch numbering.  Bit-exact, no tolerance."""
import os

import numpy as np
import pytest
import torch

from tests.golden import make_mx_reference_golden as G
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16

pytestmark = pytest.mark.gpu

_PATH = os.path.join(os.path.dirname(__file__), "golden", "mxfp4_reference_kernels_golden.npz")
GOLD = np.load(_PATH) if os.path.exists(_PATH) else None


def _numbered(case):
    """Does this call take a launch number of the row + column stochastic quantiser (mxfp4_v4/tk_quantize.cu:2853-2860)?"""
    _, fn, _, extra = case
    if not fn.startswith("mxfp4_quantize_row_and_col_opt"):
        return False
    data_sr, scale_sr = extra[1], extra[2]
    with_sign = len(extra) == 7 and extra[4]
    return bool(data_sr or scale_sr or with_sign)


@pytest.mark.skipif(GOLD is None, reason="fixture not recorded")
@pytest.mark.parametrize("idx", range(len(G.CASES)), ids=[c[0] for c in G.CASES])
def test_mxfp4_producers_reproduce_the_reference_kernels_bytes(idx):
    name, fn, kind, extra = G.CASES[idx]
    mxq = mod("mxfp4_quant_v4")
    tensors = [to_dev_bf16(a) for a in G.make_inputs(kind, 300 + idx)]
    mxq.mxfp4_set_forward_sr_invocation_count(sum(_numbered(c) for c in G.CASES[:idx]))
    r = getattr(mxq, fn)(*tensors, *extra)
    torch.cuda.synchronize()
    checked = 0
    for j, t in enumerate(r):
        key = f"{name}.{j}"
        if key not in GOLD.files:
            continue
        want = GOLD[key]
        got = t if t.dtype in (torch.float32, torch.uint8) else t.view(torch.uint8)
        got = got.cpu().numpy()
        assert got.size == want.size, key
        if got.dtype == np.float32:
            assert np.array_equal(got.reshape(-1), want.reshape(-1)), key
        else:
            bad = int((got.reshape(-1) != want.reshape(-1)).sum())
            assert bad == 0, f"{key}: {bad} of {got.size} bytes differ from the reference kernel's"
        checked += 1
    assert checked >= 2
    assert_status_ok()


@pytest.mark.skipif(GOLD is None or "gemm_0.d" not in (GOLD.files if GOLD is not None else ()), reason="fixture not recorded")
@pytest.mark.parametrize("idx", range(len(G.GEMM_SHAPES)))
def test_mxfp4_gemm_reproduces_the_reference_kernels_bytes(idx):
    """mxfp4_gemm and mxfp4_gemm_residual on operands quantised in mode 1: the bf16 outputs of the reference's compiled
    `_C_mx` kernels, bit for bit (same tcgen05 instruction, same 1/36 epilogue, one rounding)."""
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    shape = G.GEMM_SHAPES[idx]
    a, b = (to_dev_bf16(t) for t in G.gemm_operands(shape, 700 + idx))
    qa, qb = mxq.mxfp4_quantize_for_gemm(a, 1), mxq.mxfp4_quantize_for_gemm(b, 1)
    d = torch.empty(shape[0], shape[1], dtype=torch.bfloat16, device="cuda")
    gemm.mxfp4_gemm(qa[0], qa[1], qb[0], qb[1], d)
    torch.cuda.synchronize()
    assert np.array_equal(d.view(torch.int16).cpu().numpy(), GOLD[f"gemm_{idx}.d"])
    r = (0.5 * torch.randn(shape[0], shape[1], generator=torch.Generator().manual_seed(800 + idx))).to(torch.bfloat16).cuda()
    gemm.mxfp4_gemm_residual(qa[0], qa[1], qb[0], qb[1], r, d)
    torch.cuda.synchronize()
    assert np.array_equal(d.view(torch.int16).cpu().numpy(), GOLD[f"gemm_{idx}.d_residual"])
    assert_status_ok()


@pytest.mark.skipif(GOLD is None or "onepass.d" not in (GOLD.files if GOLD is not None else ()), reason="fixture not recorded")
def test_mxfp4_onepass_split2_dgrad_and_batched_gemm_reproduce_the_reference_kernels_bytes():
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    Mo, No, w = G.ONEPASS
    g1, g2 = ((torch.from_numpy(G.gemm_operands((Mo, 1, w), 720 + i)[0] * 1e-3).to(torch.bfloat16).cuda()) for i in range(2))
    q1, q2 = mxq.mxfp4_quantize_for_gemm(g1, 1), mxq.mxfp4_quantize_for_gemm(g2, 1)
    a_full = torch.cat([q1[0].view(torch.uint8), q2[0].view(torch.uint8)], dim=1).contiguous()
    ws = [mxq.mxfp4_quantize_for_gemm(to_dev_bf16(G.gemm_operands((1, No, w), 730 + i)[1]), 1) for i in range(2)]
    d = torch.empty(Mo, No, dtype=torch.bfloat16, device="cuda")
    gemm.mxfp4_split2_dgrad_strided_onepass_gemm(a_full.view(torch.float4_e2m1fn_x2), [q1[1], q2[1]], [0, w // 2], [w // 2, w // 2],
                                                 [ws[0][0], ws[1][0]], [ws[0][1], ws[1][1]], d, -1)
    torch.cuda.synchronize()
    assert np.array_equal(d.view(torch.int16).cpu().numpy(), GOLD["onepass.d"])
    d1, d2 = torch.empty_like(d), torch.empty_like(d)
    gemm.mxfp4_batched_gemm([q1[0], q2[0]], [q1[1], q2[1]], [ws[0][0], ws[1][0]], [ws[0][1], ws[1][1]], [d1, d2])
    torch.cuda.synchronize()
    assert np.array_equal(d1.view(torch.int16).cpu().numpy(), GOLD["batched.0"])
    assert np.array_equal(d2.view(torch.int16).cpu().numpy(), GOLD["batched.1"])
    assert_status_ok()


@pytest.mark.skipif(GOLD is None or "onepass_combined.d" not in (GOLD.files if GOLD is not None else ()), reason="fixture not recorded")
def test_combined_producer_into_onepass_dgrad_reproduces_the_reference_kernels_bytes():
    """The reference's call pattern for the gate/up dgrad: the combined SiLU-derivative producer's side-by-side row
    operand, and column slices (non-contiguous views) of its scale tensor, into the one-pass split GEMM."""
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    Mo, No, w = G.ONEPASS
    dh, h13 = (to_dev_bf16(t) for t in G.combined_inputs())
    q = mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col_strided_combined(dh, h13, w, w, 1)
    ws = [mxq.mxfp4_quantize_for_gemm(to_dev_bf16(G.gemm_operands((1, No, w), 730 + i)[1]), 1) for i in range(2)]
    d = torch.empty(Mo, No, dtype=torch.bfloat16, device="cuda")
    gemm.mxfp4_split2_dgrad_strided_onepass_gemm(q[0], [q[1].narrow(1, 0, w // 128), q[1].narrow(1, w // 128, w // 128)],
                                                 [0, w // 2], [w // 2, w // 2], [ws[0][0], ws[1][0]], [ws[0][1], ws[1][1]], d, -1)
    torch.cuda.synchronize()
    assert np.array_equal(d.view(torch.int16).cpu().numpy(), GOLD["onepass_combined.d"])
    # and the combined layout holds exactly the stacked producer's operands
    st = mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col(dh, h13[:, w:].contiguous(), h13[:, :w].contiguous(), 1)
    row = q[0].view(torch.uint8)
    assert torch.equal(row[:, :w // 2], st[0].view(torch.uint8)[0]) and torch.equal(row[:, w // 2:], st[0].view(torch.uint8)[1])
    assert torch.equal(q[1][:, :w // 128], st[1][0]) and torch.equal(q[1][:, w // 128:], st[1][1])
    assert torch.equal(q[2].view(torch.uint8), st[2].view(torch.uint8).reshape(2 * w, Mo // 2))
    assert torch.equal(q[3], st[3].reshape(2 * w // 128, Mo // 128, 32, 16))
    # the default producer of that GEMM: the same row operand, column operands in tensors of their own
    sp = mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols(dh, h13[:, w:].contiguous(), h13[:, :w].contiguous(), 1)
    assert torch.equal(sp[0].view(torch.uint8), row) and torch.equal(sp[1], q[1])
    for i in range(2):
        assert torch.equal(sp[2 + 2 * i].view(torch.uint8), st[2].view(torch.uint8)[i]) and torch.equal(sp[3 + 2 * i], st[3][i])
    d2 = torch.empty_like(d)
    gemm.mxfp4_split2_dgrad_strided_onepass_gemm(sp[0], [sp[1].narrow(1, 0, w // 128), sp[1].narrow(1, w // 128, w // 128)],
                                                 [0, w // 2], [w // 2, w // 2], [ws[0][0], ws[1][0]], [ws[0][1], ws[1][1]], d2, -1)
    assert torch.equal(d2, d)
    with pytest.raises(RuntimeError):
        gemm.mxfp4_split2_dgrad_strided_onepass_gemm(sp[0], [sp[1][:, :, :16], sp[1].narrow(1, w // 128, w // 128)],
                                                     [0, w // 2], [w // 2, w // 2], [ws[0][0], ws[1][0]], [ws[0][1], ws[1][1]], d2, -1)
    assert_status_ok()


@pytest.mark.skipif(GOLD is None or "onepass_split3.d" not in (GOLD.files if GOLD is not None else ()), reason="fixture not recorded")
def test_split3_quantiser_into_three_split_onepass_dgrad_reproduces_the_reference_kernels_bytes():
    """QKV dgrad as the reference runs it: dQ | dK | dV quantised without a concatenation, then one GEMM over the three
    column slices, each against its own weight operand; and the split quantisers equal the quantiser of the
    concatenation."""
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    Mo, No, _ = G.ONEPASS
    gs = [to_dev_bf16(t) for t in G.split3_inputs()]
    q = mxq.mxfp4_quantize_split3_row_and_col(*gs, 1)
    ws = [mxq.mxfp4_quantize_for_gemm(to_dev_bf16(G.gemm_operands((1, No, t.shape[1]), 750 + i)[1]), 1) for i, t in enumerate(gs)]
    offs, a_scs, off = [], [], 0
    for t in gs:
        offs.append(off // 2)
        a_scs.append(q[1].narrow(1, off // 128, t.shape[1] // 128))
        off += t.shape[1]
    d = torch.empty(Mo, No, dtype=torch.bfloat16, device="cuda")
    gemm.mxfp4_split3_dgrad_strided_onepass_gemm(q[0], a_scs, offs, [t.shape[1] // 2 for t in gs], [x[0] for x in ws],
                                                 [x[1] for x in ws], d, -1)
    torch.cuda.synchronize()
    assert np.array_equal(d.view(torch.int16).cpu().numpy(), GOLD["onepass_split3.d"])
    whole = mxq.mxfp4_quantize_row_and_col(torch.cat(gs, 1).contiguous(), 1)
    for a, b in zip(q, whole):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    two = mxq.mxfp4_quantize_split2_row_and_col(gs[0], gs[1], 1)
    whole2 = mxq.mxfp4_quantize_row_and_col(torch.cat(gs[:2], 1).contiguous(), 1)
    for a, b in zip(two, whole2):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    outs = [torch.empty_like(t) for t in q]
    assert mxq.mxfp4_quantize_split3_row_and_col_launch_inplace(*gs, *outs, 1) is None
    for a, b in zip(outs, q):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    with pytest.raises(RuntimeError):
        mxq.mxfp4_quantize_split3_row_and_col(gs[0], gs[1], gs[2][:128], 1)
    assert_status_ok()


def test_nhsd_attention_output_quantiser_equals_the_quantiser_of_the_transposed_copy():
    mxq = mod("mxfp4_quant_v4")
    g = torch.Generator(device="cuda").manual_seed(5)
    for shape in ((2, 8, 256, 64), (1, 4, 384, 128)):
        x = torch.randn(*shape, device="cuda", generator=g).to(torch.bfloat16)
        B, H, S, D = shape
        flat = x.permute(0, 2, 1, 3).reshape(B * S, H * D).contiguous()
        for a, b in zip(mxq.mxfp4_quantize_nhsd_wo_row_and_col(x, 1), mxq.mxfp4_quantize_row_and_col(flat, 1)):
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    with pytest.raises(RuntimeError):
        mxq.mxfp4_quantize_nhsd_wo_row_and_col(x[:, :, :64].contiguous(), 1)      # S not a multiple of 128
    with pytest.raises(RuntimeError):
        mxq.mxfp4_quantize_nhsd_wo_row_and_col(torch.zeros(1, 4, 128, 32, dtype=torch.bfloat16, device="cuda"), 1)
    assert_status_ok()


@pytest.mark.skipif(GOLD is None or "split3_inverse_rope.0" not in (GOLD.files if GOLD is not None else ()), reason="fixture not recorded")
def test_split3_quantiser_with_the_inverse_rotation_folded_in_reproduces_the_reference_kernels_bytes():
    """dQ and dK rotated back on the way into the quantiser (heads of 64), dV as it is: the reference kernel's bytes, and
    the same bytes as the separate inverse-rotation kernel followed by the split quantiser."""
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c")
    gs, cs = G.inverse_rope_inputs()
    dev = [to_dev_bf16(t) for t in gs]
    cs_dev = torch.from_numpy(cs).cuda()
    r = mxq.mxfp4_quantize_split3_row_and_col_inverse_rope_live64(*dev, cs_dev, cs.shape[0], 1)
    torch.cuda.synchronize()
    for j, t in enumerate(r):
        bad = int((t.view(torch.uint8).cpu().numpy().reshape(-1) != GOLD[f"split3_inverse_rope.{j}"].reshape(-1)).sum())
        assert bad == 0, f"output {j}: {bad} bytes differ from the reference kernel's"
    q_rot, k_rot = torch.empty_like(dev[0]), torch.empty_like(dev[1])
    gemm.nvfp4_inverse_rope_packed_qk(dev[0], dev[1], cs_dev, cs.shape[0], 64, q_rot, k_rot)
    for a, b in zip(r, mxq.mxfp4_quantize_split3_row_and_col(q_rot, k_rot, dev[2], 1)):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    with pytest.raises(RuntimeError):
        mxq.mxfp4_quantize_split3_row_and_col_inverse_rope_live64(*dev, cs_dev[:, :16].contiguous(), cs.shape[0], 1)
    assert_status_ok()


@pytest.mark.skipif(GOLD is None or "gemm_rope64.d" not in (GOLD.files if GOLD is not None else ()), reason="fixture not recorded")
@pytest.mark.parametrize("tag,idx,pair_dim", [("rope64", 0, 32), ("rope128", 1, 64)])
def test_mxfp4_gemm_with_rotary_epilogue_reproduces_the_reference_kernels_bytes(tag, idx, pair_dim):
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    shape = G.GEMM_SHAPES[idx]
    a, b = (to_dev_bf16(t) for t in G.gemm_operands(shape, 780))
    qa, qb = mxq.mxfp4_quantize_for_gemm(a, 1), mxq.mxfp4_quantize_for_gemm(b, 1)
    cs = torch.from_numpy(G.rope_table(128, pair_dim)).cuda()
    d = torch.empty(shape[0], shape[1], dtype=torch.bfloat16, device="cuda")
    gemm.mxfp4_gemm_rope_live64(qa[0], qa[1], qb[0], qb[1], d, cs, 128)
    torch.cuda.synchronize()
    assert np.array_equal(d.view(torch.int16).cpu().numpy(), GOLD[f"gemm_{tag}.d"])
    d2 = torch.empty_like(d)
    gemm.mxfp4_gemm_rope_live_config(qa[0], qa[1], qb[0], qb[1], d2, cs, 128, 3)
    assert torch.equal(d2, d)
    if f"gemm_{tag}.d_tables" in GOLD.files:      # separate cos / sin tables, full rotation
        gemm.mxfp4_gemm_rope(qa[0], qa[1], qb[0], qb[1], d2, cs[..., 0].contiguous(), cs[..., 1].contiguous(), 128,
                             2 * pair_dim, 2 * pair_dim)
        torch.cuda.synchronize()
        assert np.array_equal(d2.view(torch.int16).cpu().numpy(), GOLD[f"gemm_{tag}.d_tables"])
        with pytest.raises(RuntimeError):
            gemm.mxfp4_gemm_rope(qa[0], qa[1], qb[0], qb[1], d2, cs[..., 0].contiguous(), cs[..., 1].contiguous(), 128,
                                 2 * pair_dim, pair_dim)
    with pytest.raises(RuntimeError):
        gemm.mxfp4_gemm_rope_live64(qa[0], qa[1], qb[0], qb[1], d, cs, 96)
    assert_status_ok()


@pytest.mark.skipif(GOLD is None or "batched_rope.0" not in (GOLD.files if GOLD is not None else ()), reason="fixture not recorded")
def test_mxfp4_batched_qkv_projection_with_rotary_epilogue_reproduces_the_reference_kernels_bytes():
    """One activation against three weights, Q and K rotated in the epilogue, V not (its table is empty)."""
    mxq, gemm = mod("mxfp4_quant_v4"), mod("tk_gemm_c_mx")
    shape = G.GEMM_SHAPES[0]
    qa = mxq.mxfp4_quantize_for_gemm(to_dev_bf16(G.gemm_operands(shape, 781)[0]), 1)
    ws = [mxq.mxfp4_quantize_for_gemm(to_dev_bf16(G.gemm_operands(shape, 782 + i)[1]), 1) for i in range(3)]
    cs = torch.from_numpy(G.rope_table(128, 32)).cuda()
    ds = [torch.empty(shape[0], shape[1], dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    gemm.mxfp4_batched_gemm_rope_live64([qa[0]] * 3, [qa[1]] * 3, [w[0] for w in ws], [w[1] for w in ws], ds,
                                        [cs, cs, torch.empty(0, dtype=torch.float32, device="cuda")], [128, 128, 0])
    torch.cuda.synchronize()
    for i, d in enumerate(ds):
        assert np.array_equal(d.view(torch.int16).cpu().numpy(), GOLD[f"batched_rope.{i}"]), i
    assert_status_ok()
