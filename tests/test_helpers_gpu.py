"""GPU parity of the entry points around the hot path: element-wise fp32 <-> packed E2M1, the GEMM
module's own tile quantiser, the reduction of GEMM-epilogue row partials into 1/rms (and the fused
producers fed by it), the MXFP4 32x32 weight quantiser, the batched quantiser."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16, u8

pytestmark = pytest.mark.gpu


def test_fp32_fp4x2_round_trip():
    gemm = mod("tk_gemm_c")
    rng = np.random.default_rng(11)
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 100.0, 0.0, -0.0, -0.25, -2.5, -5.0, -9.0],
                    dtype=np.float32)
    x = np.concatenate([ties, (rng.standard_normal(4096 - ties.size) * 3).astype(np.float32)]).reshape(64, 64)
    packed = gemm.fp32_to_fp4x2(torch.from_numpy(x).cuda())
    assert packed.dtype == torch.float4_e2m1fn_x2 and tuple(packed.shape) == (64, 32)
    ref = o.pack_fp4(o.e2m1_encode_rn(x))
    assert np.array_equal(u8(packed), ref)
    back = gemm.fp4x2_to_fp32(packed).cpu().numpy()
    assert np.array_equal(back.view(np.uint32), o.E2M1_TO_F32[o.unpack_fp4(ref)].astype(np.float32).view(np.uint32))
    assert_status_ok()


@pytest.mark.parametrize("scale_2d", [False, True])
@pytest.mark.parametrize("shape", [(128, 128), (256, 512)])
def test_gemm_module_quantiser(shape, scale_2d):
    gemm = mod("tk_gemm_c")
    M, N = shape
    a = o.make_activations(M, N, seed=M + N + int(scale_2d))
    a[3, 16:32] = 0.0
    fp4 = torch.empty((M, N // 2), dtype=torch.uint8, device="cuda")
    sc = torch.empty((M // 128, N // 64, 512), dtype=torch.uint8, device="cuda")
    sg = torch.full((1,), 123.0, dtype=torch.float32, device="cuda")
    gemm.nvfp4_quantize(to_dev_bf16(a), fp4.view(torch.float4_e2m1fn_x2), sc.view(torch.float8_e4m3fn), sg, scale_2d)
    torch.cuda.synchronize()
    ref = o.tk_nvfp4_quantize(a, scale_2d)
    assert sg.item() == ref["sg"]
    assert np.array_equal(u8(sc).reshape(ref["sc"].shape), ref["sc"])
    assert np.array_equal(u8(fp4), ref["fp4"])
    assert_status_ok()


def _partials(x, group):
    M, K = x.shape
    return (x.astype(np.float32) ** 2).reshape(M, K // group, group).sum(axis=-1, dtype=np.float32)


@pytest.mark.parametrize("shape", [(128, 512), (256, 4096)])
def test_row_rms_reduce_and_fused_from_partials(shape):
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    M, K = shape
    x = o.make_activations(M, K, seed=K + 3)
    g = o.make_gamma(K, seed=K + 4)
    part = _partials(x, 32)
    ref_inv = o.row_rms_reduce(part, K, 1e-5)
    p_dev = torch.from_numpy(part).cuda()
    coeff = torch.empty(M, dtype=torch.float32, device="cuda")
    gemm.nvfp4_row_rms_reduce(p_dev, coeff, K, 1e-5)
    inv = coeff.cpu().numpy()
    assert np.abs(inv / ref_inv - 1).max() < 2e-6   # hardware rsqrtf vs the correctly rounded value
    out = tkq.tk_fused_norm_quantize_from_row_rms_partial(to_dev_bf16(x), to_dev_bf16(g), p_dev, 1e-5, False, True)
    torch.cuda.synchronize()
    assert torch.equal(out[5], coeff)
    ref = o.nvfp4_fused_norm_quantize(x, g, 1e-5, inv_rms=inv)
    for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
        assert np.array_equal(u8(out[i]).reshape(ref[k].shape), ref[k]), k
    with pytest.raises(RuntimeError):
        gemm.nvfp4_row_rms_reduce(torch.zeros((M, 7), device="cuda"), coeff, K, 1e-5)   # 7 does not divide K
    assert_status_ok()


def test_mxfp4_weight_2d_and_from_partials():
    mxq = mod("mxfp4_quant_v4")
    N, K = 256, 384
    w = o.bf16_round((0.02 * np.random.default_rng(7).standard_normal((N, K))).astype(np.float32))
    w[:32, :32] = 0.0                      # an all-zero tile: scale byte 0
    w[32:64, 32:64] *= 0.87 / np.abs(w[32:64, 32:64]).max() * 2.0 ** -6   # amax close to the 0.87 threshold
    w = o.bf16_round(w)
    out = mxq.mxfp4_quantize_weight_2d(to_dev_bf16(w))
    torch.cuda.synchronize()
    ref = o.mxfp4_quantize_weight_2d(w)
    for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
        assert np.array_equal(u8(out[i]).reshape(ref[k].shape), ref[k]), k
    # both exponents of the rule occur in this weight
    lowered = ref["row_sc_logical"] != o.mx_e8m0(np.repeat(np.abs(w).reshape(N // 32, 32, K // 32, 32).max(axis=(1, 3)), 32, axis=0), 1)
    assert lowered.any() and not lowered.all()

    M, Kx = 256, 4096
    x = o.make_activations(M, Kx, seed=77)
    g = o.make_gamma(Kx, seed=78)
    part = torch.from_numpy(_partials(x, 256)).cuda()
    res = mxq.mxfp4_fused_rmsnorm_quantize_row_and_col_from_row_rms_partial(to_dev_bf16(x), to_dev_bf16(g), part, 1e-5, 1)
    torch.cuda.synchronize()
    inv = res[4].cpu().numpy()
    assert np.abs(inv / o.row_rms_reduce(part.cpu().numpy(), Kx, 1e-5) - 1).max() < 2e-6
    refq = o.mxfp4_quantize_row_and_col(o.rmsnorm_apply(x, inv, g), 1)
    for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
        assert np.array_equal(u8(res[i]).reshape(refq[k].shape), refq[k]), k
    with pytest.raises(RuntimeError):
        mxq.mxfp4_fused_rmsnorm_quantize_row_and_col_from_row_rms_partial(to_dev_bf16(x), to_dev_bf16(g), part, 1e-5, 0)
    assert_status_ok()


def test_batched_quantize_matches_single_calls():
    tkq = mod("tk_quant_v5")
    xs = [to_dev_bf16(o.make_activations(128 * (i + 1), 256, seed=90 + i)) for i in range(3)]
    lists = tkq.tk_batched_quantize_for_gemm(xs, True, True)
    assert len(lists) == 8 and all(len(l) == 3 for l in lists)
    for i, x in enumerate(xs):
        single = tkq.tk_quantize_for_gemm(x, True, True)
        torch.cuda.synchronize()
        for j in range(4):
            assert torch.equal(lists[j][i].view(torch.uint8), single[j].view(torch.uint8))
        assert torch.equal(lists[4][i], single[4])
    assert_status_ok()


def test_mxfp4_silu_deriv_split2():
    mxq, tkq = mod("mxfp4_quant_v4"), mod("tk_quant_v5")
    M, H = 256, 384
    rng = np.random.default_rng(21)
    dh = o.bf16_round((1e-3 * rng.standard_normal((M, H))).astype(np.float32))
    h3 = o.bf16_round(rng.standard_normal((M, H)).astype(np.float32))
    h1 = o.bf16_round((2.0 * rng.standard_normal((M, H))).astype(np.float32))
    out = mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col(to_dev_bf16(dh), to_dev_bf16(h3), to_dev_bf16(h1), 1)
    assert tuple(out[0].shape) == (2, M, H // 2) and tuple(out[3].shape) == (2, H // 128, M // 128, 32, 16)
    dh1, dh3 = tkq.tk_silu_deriv_split_bf16(to_dev_bf16(dh), to_dev_bf16(h3), to_dev_bf16(h1))
    torch.cuda.synchronize()
    # the derivative itself (hardware __expf) is checked against the oracle in the NVFP4 SwiGLU tests
    for i, t in enumerate((dh1, dh3)):
        ref = o.mxfp4_quantize_row_and_col(t.float().cpu().numpy(), 1)
        for j, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
            assert np.array_equal(u8(out[j][i]).reshape(ref[k].shape), ref[k]), (i, k)
    assert_status_ok()


@pytest.mark.parametrize("head", [64, 128])
def test_rope_packed_qk_forward_and_inverse(head):
    """Rotary embedding of Q and K in one launch, both directions bit-exact against the oracle; the inverse undoes
    the forward up to the two bf16 roundings."""
    gemm = mod("tk_gemm_c")
    rows, seq, q_dim, k_dim = 512, 128, 4 * head, head
    rng = np.random.default_rng(head)
    q = o.bf16_round(rng.standard_normal((rows, q_dim)).astype(np.float32))
    k = o.bf16_round(rng.standard_normal((rows, k_dim)).astype(np.float32))
    ang = rng.uniform(0, 2 * np.pi, size=(seq, head // 2)).astype(np.float32)
    cs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)
    qd, kd, csd = to_dev_bf16(q), to_dev_bf16(k), torch.from_numpy(cs).cuda()
    qf, kf = torch.empty_like(qd), torch.empty_like(kd)
    gemm.nvfp4_forward_rope_packed_qk(qd, kd, csd, seq, head, qf, kf)
    qi, ki = torch.empty_like(qd), torch.empty_like(kd)
    gemm.nvfp4_inverse_rope_packed_qk(qf, kf, csd, seq, head, qi, ki)
    torch.cuda.synchronize()
    ref_qf, ref_kf = o.rope_packed(q, cs, False), o.rope_packed(k, cs, False)
    assert np.array_equal(qf.float().cpu().numpy(), ref_qf) and np.array_equal(kf.float().cpu().numpy(), ref_kf)
    assert np.array_equal(qi.float().cpu().numpy(), o.rope_packed(ref_qf, cs, True))
    assert np.array_equal(ki.float().cpu().numpy(), o.rope_packed(ref_kf, cs, True))
    assert np.abs(qi.float().cpu().numpy() - q).max() <= 2.0 ** -6 * np.abs(q).max()
    with pytest.raises(RuntimeError):
        gemm.nvfp4_forward_rope_packed_qk(qd, kd, csd, seq, head, qd, kf)          # output aliases an input
    with pytest.raises(RuntimeError):
        gemm.nvfp4_forward_rope_packed_qk(qd, kd, csd[:96].contiguous(), 96, head, qf, kf)   # not a power of two
    assert_status_ok()


def test_a_bounded_wait_that_runs_out_reports_through_the_status_word():
    """No kernel of the library spins without a limit: a wait that runs out stores a code in the device's status
    word and the kernel returns.  The self-test kernel makes that happen harmlessly (a barrier nobody arrives on,
    ~50 us limit); the host then reads the code once, and 0 afterwards, and the context stays usable."""
    lib = mod("_lib")
    assert lib.device_status() == 0
    lib.call("fp4b200_selftest_bounded_wait", 100000, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert lib.device_status() == 6          # kStatusSelfTestTimeout; reading clears the word
    assert lib.device_status() == 0
    x = torch.ones(8, device="cuda")
    assert (x + 1).sum().item() == 16.0      # the context is alive
    with pytest.raises(RuntimeError, match="1 to 1e8"):
        lib.call("fp4b200_selftest_bounded_wait", 0, None)
