"""GPU parity: NVFP4 producers through the reference-shaped shim (and so through the C ABI)
against the CPU oracle on identical seeded inputs.  Codes and scale bytes must be bit-exact."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16, u8

pytestmark = pytest.mark.gpu


def _check_operands(out, ref, want_col=True):
    assert np.array_equal(u8(out[0]), ref["row_fp4"]), "row codes differ"
    assert np.array_equal(u8(out[1]).reshape(ref["row_sc"].shape), ref["row_sc"]), "row scales differ"
    if want_col:
        assert np.array_equal(u8(out[2]), ref["col_fp4"]), "column codes differ"
        assert np.array_equal(u8(out[3]).reshape(ref["col_sc"].shape), ref["col_sc"]), "column scales differ"


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (1024, 512), (384, 4096), (2048, 4096)])
@pytest.mark.parametrize("ec", [True, False])
def test_quantize_for_gemm_bit_exact(shape, ec):
    tkq = mod("tk_quant_v5")
    x = o.make_activations(*shape, seed=shape[0] + shape[1])
    out = tkq.tk_quantize_for_gemm(to_dev_bf16(x), True, ec)
    torch.cuda.synchronize()
    ref = o.nvfp4_quantize_for_gemm(x, True, ec)
    _check_operands(out, ref)
    assert out[4].item() == ref["sg"] and out[6][0].item() == ref["amax"]
    assert out[0].dtype == torch.float4_e2m1fn_x2 and out[1].dtype == torch.float8_e4m3fn
    assert tuple(out[1].shape) == (shape[0] // 128, shape[1] // 64, 512)
    assert_status_ok()


@pytest.mark.parametrize("ec", [True, False])
@pytest.mark.parametrize("amax_exp", [0, 7, -20, 100])
def test_block_scale_for_every_bf16_block_maximum(amax_exp, ec):
    """Every positive bf16 value of 24 binades below the tensor amax is the maximum of some 16-block: the scale
    byte for all of them, normal and subnormal E4M3 results, saturation and the tiny-amax branch, in both passes."""
    tkq = mod("tk_quant_v5")
    top = 127 + amax_exp                                   # biased exponent of the tensor amax 2^amax_exp
    expo = np.arange(top - 24, top, dtype=np.uint32)
    expo = expo[(expo >= 1) & (expo <= 254)]
    bits = ((expo[:, None] << 7) | np.arange(128, dtype=np.uint32)[None, :]).reshape(-1).astype(np.uint16)
    vals = o.bf16_from_bits(bits)                          # ascending positive bf16 values
    n_blocks = (-(-vals.size // 2048)) * 2048
    v = np.resize(vals, n_blocks)
    M, K = 128, n_blocks * 16 // 128
    rng = np.random.default_rng(amax_exp + 1000)
    x = (rng.uniform(-1, 1, size=(n_blocks, 16)).astype(np.float32) * v[:, None])
    x[:, 3] = v * np.where(rng.integers(0, 2, size=n_blocks) == 0, 1.0, -1.0)   # the block maximum itself
    x = o.bf16_round(x).reshape(M, K)
    x[0, 0] = np.float32(2.0 ** amax_exp)
    out = tkq.tk_quantize_for_gemm(to_dev_bf16(x), True, ec)
    torch.cuda.synchronize()
    ref = o.nvfp4_quantize_for_gemm(x, True, ec)
    _check_operands(out, ref)
    assert_status_ok()


def test_quantize_row_only_and_golden_inputs(golden):
    tkq = mod("tk_quant_v5")
    x = o.bf16_from_bits(golden["mid_x_bits"])
    out = tkq.tk_quantize_for_gemm(to_dev_bf16(x), False, False)
    torch.cuda.synchronize()
    assert out[2].numel() == 0 and out[3].numel() == 0
    # decode-centric codes/scales equal the bytes the reference's CPU emulation produced
    assert np.array_equal(u8(out[0]), golden["mid_ec_x_data"])
    assert np.array_equal(o.unswizzle_scales(u8(out[1]), 256, 32), golden["mid_ec_x_scale"])
    assert_status_ok()


def test_edge_values_zero_blocks_and_negative_zero():
    tkq = mod("tk_quant_v5")
    x = o.make_activations(256, 256, seed=5)
    x[:16, :32] = 0.0            # all-zero blocks in both orientations
    x[40, 64:80] = -0.0          # negative zeros keep their sign bit in the code
    x[100:116, 200] = 1e-30      # tiny block amax
    x[200, 0] = 3.0e38           # huge outlier -> S_enc tiny
    x = o.bf16_round(x)
    for ec in (True, False):
        out = tkq.tk_quantize_for_gemm(to_dev_bf16(x), True, ec)
        torch.cuda.synchronize()
        _check_operands(out, o.nvfp4_quantize_for_gemm(x, True, ec))
    z = np.zeros((128, 128), dtype=np.float32)
    out = tkq.tk_quantize_for_gemm(to_dev_bf16(z), True, True)
    torch.cuda.synchronize()
    _check_operands(out, o.nvfp4_quantize_for_gemm(z, True, True))
    assert out[4].item() == 0.0
    assert_status_ok()


@pytest.mark.parametrize("shape", [(128, 128), (256, 640), (512, 2048), (1024, 4096), (256, 8192)])
def test_fused_norm_quantize(shape):
    tkq = mod("tk_quant_v5")
    M, K = shape
    x = o.make_activations(M, K, seed=M * 3 + K)
    g = o.make_gamma(K, seed=K)
    out = tkq.tk_fused_norm_quantize(to_dev_bf16(x), to_dev_bf16(g), 1e-5, False, True)
    torch.cuda.synchronize()
    inv_gpu = out[5].cpu().numpy()
    inv_ref = o.rmsnorm_inv_rms(x, 1e-5)
    # rsqrtf is a hardware approximation: tolerance 2e-6 relative, as in the reference's own test
    assert np.abs(inv_gpu / inv_ref - 1).max() < 2e-6
    # bit-exact given the GPU's inverse RMS
    ref = o.nvfp4_fused_norm_quantize(x, g, 1e-5, inv_rms=inv_gpu)
    _check_operands(out, ref)
    # properties the reference's GPU test pins: amax identity and sg == amax/2688
    assert out[6].item() == ref["amax"]
    assert out[4].item() == np.float32(ref["amax"] / np.float32(2688.0))
    assert_status_ok()


def test_fused_norm_from_inv_rms_bit_exact_vs_pure_oracle():
    """With a shared inverse RMS the whole producer is reproducible on the CPU."""
    tkq = mod("tk_quant_v5")
    M, K = 512, 1024
    x = o.make_activations(M, K, seed=77)
    g = o.make_gamma(K, seed=78)
    inv = o.rmsnorm_inv_rms(x, 1e-5)
    out = tkq.tk_fused_norm_quantize_from_inv_rms(to_dev_bf16(x), to_dev_bf16(g),
                                                  torch.from_numpy(inv).cuda(), False, True)
    torch.cuda.synchronize()
    _check_operands(out, o.nvfp4_fused_norm_quantize(x, g, 1e-5, inv_rms=inv))
    assert out[5].data_ptr() != 0 and np.array_equal(out[5].cpu().numpy(), inv)
    assert_status_ok()


def test_full_size_properties_config2():
    """Benchmark-size case (16384 x 4096): size-independent properties instead of a full oracle run —
    determinism, a sampled-row oracle check, column codes equal to the row codes of the
    transposed input."""
    tkq = mod("tk_quant_v5")
    M, K = 16384, 4096
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    x[:, torch.randperm(K, generator=gen)[:4]] *= 20
    g = (1 + 0.1 * torch.randn(K, generator=gen)).to(torch.bfloat16)
    xd, gd = x.cuda(), g.cuda()
    a = tkq.tk_fused_norm_quantize(xd, gd, 1e-5, False, True)
    b = tkq.tk_fused_norm_quantize(xd, gd, 1e-5, False, True)
    torch.cuda.synchronize()
    for i in range(4):
        assert torch.equal(a[i].view(torch.uint8), b[i].view(torch.uint8))
    inv = a[5].cpu().numpy()
    xf = x.float().numpy()
    n = o.rmsnorm_apply(xf, inv, g.float().numpy())
    assert a[6].item() == np.abs(n).max()
    rows = np.arange(0, M, 128 * 17)[:6]
    for r0 in rows:
        blk = n[r0:r0 + 128]
        codes, sc = o.nvfp4_quantize_1d(blk, a[6].item(), "encode")
        assert np.array_equal(u8(a[0][r0:r0 + 128]), codes)
        assert np.array_equal(u8(a[1][r0 // 128]).reshape(-1), o.swizzle_scales(sc).reshape(-1))
        ccodes, csc = o.nvfp4_quantize_1d(np.ascontiguousarray(blk.T), a[6].item(), "encode")
        assert np.array_equal(u8(a[2][:, r0 // 2:(r0 + 128) // 2]), ccodes)
    assert_status_ok()


@pytest.mark.parametrize("shape", [(128, 128), (512, 1024), (1792, 4096)])
def test_quantize_weight_2d(shape):
    tkq = mod("tk_quant_v5")
    N, K = shape
    w = o.bf16_round((0.02 * np.random.default_rng(N).standard_normal((N, K))).astype(np.float32))
    w[:16, :16] = 0.0
    out = tkq.tk_quantize_weight_2d(to_dev_bf16(w))
    torch.cuda.synchronize()
    amax = o.tensor_amax(w)
    r, rs, c, cs = o.nvfp4_quantize_2d(w, amax)
    assert np.array_equal(u8(out[0]), r) and np.array_equal(u8(out[2]), c)
    assert np.array_equal(u8(out[1]).reshape(-1), o.swizzle_scales(rs).reshape(-1))
    assert np.array_equal(u8(out[3]).reshape(-1), o.swizzle_scales(cs).reshape(-1))
    # the property the reference relies on: column codes are the transpose of the row codes
    assert np.array_equal(o.unpack_fp4(u8(out[2])), o.unpack_fp4(u8(out[0])).T)
    assert out[4].item() == o.nvfp4_global_decode_scale(amax)
    assert_status_ok()


@pytest.mark.parametrize("ec", [True, False])
@pytest.mark.parametrize("shape", [(1, 2, 128, 64), (3, 6, 256, 64), (2, 32, 1024, 64)])
def test_quantize_nhsd_wo_equals_quantising_the_permuted_tensor(shape, ec):
    """Attention output in [B, H, S, D] layout: same bytes as quantising its [B*S, H*D] permutation, and (for the
    small shapes) as the oracle."""
    tkq = mod("tk_quant_v5")
    B, H, S, D = shape
    M, K = B * S, H * D
    x = o.make_activations(M, K, seed=B + H + S)                      # the logical matrix
    x_nhsd = np.ascontiguousarray(x.reshape(B, S, H, D).transpose(0, 2, 1, 3))
    out = tkq.tk_quantize_nhsd_wo_for_gemm(to_dev_bf16(x_nhsd), True, ec)
    flat = tkq.tk_quantize_for_gemm(to_dev_bf16(x), True, ec)
    torch.cuda.synchronize()
    for i in range(4):
        assert torch.equal(out[i].view(torch.uint8), flat[i].view(torch.uint8)), i
    assert torch.equal(out[6], flat[6])
    if M * K <= 1 << 20:
        _check_operands(out, o.nvfp4_quantize_for_gemm(x, True, ec))
    row_only = tkq.tk_quantize_nhsd_wo_for_gemm(to_dev_bf16(x_nhsd), False, ec)
    torch.cuda.synchronize()
    assert torch.equal(row_only[0].view(torch.uint8), flat[0].view(torch.uint8)) and row_only[2].numel() == 0
    with pytest.raises(RuntimeError):
        tkq.tk_quantize_nhsd_wo_for_gemm(to_dev_bf16(x_nhsd[:, :, :64]), True, ec)      # S not a multiple of 128
    with pytest.raises(RuntimeError):
        tkq.tk_quantize_nhsd_wo_for_gemm(to_dev_bf16(np.zeros((1, 2, 128, 32), np.float32)), True, ec)   # head_dim 32
    assert_status_ok()


@pytest.mark.parametrize("M,splits", [(1024, (2048, 512, 512)), (4096, (2048, 512, 512)), (128, (128, 128, 128)),
                                      (256, (4096, 128, 128)), (384, (128, 2560, 384))])
def test_split3_one_launch_equals_the_single_input_quantiser(M, splits):
    """The grouped launch (CTAs shared out among the three matrices; at M = 4096 each warp takes strip pairs) writes
    the bytes of one single-input quantiser call per stream: attention-gradient widths, one chunk per matrix, and
    very unequal widths (a matrix's share of the CTAs is never less than one)."""
    tkq = mod("tk_quant_v5")
    g = torch.Generator(device="cuda").manual_seed(M)
    xs = [(10.0 ** (-i) * torch.randn(M, n, device="cuda", generator=g)).to(torch.bfloat16) for i, n in enumerate(splits)]
    out = tkq.tk_group_quantize_dim1_split3_for_gemm(*xs)
    off = 0
    for i, (x, n) in enumerate(zip(xs, splits)):
        one = tkq.tk_quantize_for_gemm(x, True, True)
        assert torch.equal(out[0][i].contiguous().view(torch.uint8), one[0].view(torch.uint8))
        assert torch.equal(out[1][i].view(torch.uint8).flatten(), one[1].view(torch.uint8).flatten())
        assert torch.equal(out[3][i].view(torch.uint8), one[2].view(torch.uint8))
        assert torch.equal(out[4][i].view(torch.uint8).flatten(), one[3].view(torch.uint8).flatten())
        assert out[2][i].item() == one[4].item() and out[12][i].item() == x.float().abs().max().item()
        off += n
    assert out[6].is_contiguous() and out[8].is_contiguous()
    assert torch.equal(out[8].view(torch.uint8), torch.cat([t.view(torch.uint8) for t in out[4]], 0))
    assert_status_ok()


@pytest.mark.parametrize("sections", [(512, 128, 256), (256, 384), (128, 128, 256, 128)])
def test_group_quantiser_of_one_matrix_equals_the_single_input_quantiser_per_group(sections):
    """tk_group_quantize_dim1_for_gemm: the column groups of a concatenated matrix, three groups through the grouped
    launch, other counts one call per group."""
    tkq = mod("tk_quant_v5")
    M = 256
    g = torch.Generator(device="cuda").manual_seed(sum(sections))
    parts = [(10.0 ** (-i) * torch.randn(M, n, device="cuda", generator=g)).to(torch.bfloat16) for i, n in enumerate(sections)]
    out = tkq.tk_group_quantize_dim1_for_gemm(torch.cat(parts, 1).contiguous(), list(sections))
    assert len(out) == 9
    for i, x in enumerate(parts):
        one = tkq.tk_quantize_for_gemm(x, True, True)
        assert torch.equal(out[0][i].contiguous().view(torch.uint8), one[0].view(torch.uint8))
        assert torch.equal(out[1][i].view(torch.uint8).flatten(), one[1].view(torch.uint8).flatten())
        assert torch.equal(out[3][i].view(torch.uint8), one[2].view(torch.uint8))
        assert torch.equal(out[4][i].view(torch.uint8).flatten(), one[3].view(torch.uint8).flatten())
        assert out[2][i].item() == one[4].item()
    assert torch.equal(out[6].view(torch.uint8), torch.cat([t.view(torch.uint8) for t in out[1]], 1))
    assert torch.equal(out[8].view(torch.uint8), torch.cat([t.view(torch.uint8) for t in out[4]], 0))
    with pytest.raises(RuntimeError):
        tkq.tk_group_quantize_dim1_for_gemm(torch.cat(parts, 1).contiguous(), [128])
    assert_status_ok()


def test_split3_group_quantiser_writes_slices_of_the_concatenated_operands():
    """Three gradient streams of different widths (one of them a strided view), each with its own tensor amax: the
    slices of the concatenated code matrices and the per-group scales equal the single-input quantiser's bytes,
    which the oracle checks; the concatenated scale tensors are the per-group ones side by side."""
    tkq = mod("tk_quant_v5")
    M, splits = 256, (512, 128, 256)
    xs = [o.make_activations(M, n, seed=60 + i, scale=10.0 ** (-i)) for i, n in enumerate(splits)]
    wide = to_dev_bf16(np.concatenate([xs[1], xs[1]], axis=1))
    devs = [to_dev_bf16(xs[0]), wide[:, :splits[1]], to_dev_bf16(xs[2])]        # the middle input has row stride 256
    out = tkq.tk_group_quantize_dim1_split3_for_gemm(*devs)
    torch.cuda.synchronize()
    assert len(out) == 15
    rows, row_sc, sg, cols, col_sc, row_full, row_sc_cat, col_full, col_sc_cat = out[:9]
    n_total = sum(splits)
    assert tuple(row_full.shape) == (M, n_total // 2) and tuple(col_full.shape) == (n_total, M // 2)
    off = 0
    for g, (x, n) in enumerate(zip(xs, splits)):
        ref = o.nvfp4_quantize_for_gemm(x, True, True)
        assert np.array_equal(u8(rows[g]), ref["row_fp4"]) and np.array_equal(u8(cols[g]), ref["col_fp4"])
        assert np.array_equal(u8(row_sc[g]).reshape(ref["row_sc"].shape), ref["row_sc"])
        assert np.array_equal(u8(col_sc[g]).reshape(ref["col_sc"].shape), ref["col_sc"])
        assert sg[g].item() == ref["sg"] and out[12][g].item() == ref["amax"]
        assert np.array_equal(u8(row_full)[:, off // 2:(off + n) // 2], ref["row_fp4"])
        assert np.array_equal(u8(col_full)[off:off + n], ref["col_fp4"])
        assert rows[g].data_ptr() == row_full.data_ptr() + off // 2                # views of the full buffers
        off += n
    assert np.array_equal(u8(row_sc_cat), np.concatenate([u8(t) for t in row_sc], axis=1))
    assert np.array_equal(u8(col_sc_cat), np.concatenate([u8(t) for t in col_sc], axis=0))
    with pytest.raises(RuntimeError):
        tkq.tk_group_quantize_dim1_split3_for_gemm(*devs, True, 1, 0, "row")       # SR of one axis only: not built
    # stochastic rounding of both axes: one launch of the tuned kernel per stream, at consecutive invocation offsets
    tkq.tk_set_sr_invocation_count(4)
    out = tkq.tk_group_quantize_dim1_split3_for_gemm(*devs, True, 77, 3, "both")
    torch.cuda.synchronize()
    assert tkq.tk_sr_invocation_count() == 7
    off = 0
    for g, (x, n) in enumerate(zip(xs, splits)):
        amax = o.tensor_amax(x)
        ref = o.nvfp4_quantize_transpose_launch(x, amax, amax, True, True, True, False, False, True, 77, 3 + ((4 + g) << 32))
        assert np.array_equal(u8(out[5])[:, off // 2:(off + n) // 2], ref["row_fp4"])
        assert np.array_equal(u8(out[7])[off:off + n], ref["col_fp4"])
        assert np.array_equal(u8(out[1][g]).reshape(ref["row_sc"].shape), ref["row_sc"])
        assert np.array_equal(u8(out[4][g]).reshape(ref["col_sc"].shape), ref["col_sc"])
        assert out[2][g].item() == o.nvfp4_global_decode_scale(amax)
        off += n
    with pytest.raises(RuntimeError):
        tkq.tk_group_quantize_dim1_split3_for_gemm(devs[0], devs[1], to_dev_bf16(xs[2][:128]))
    assert_status_ok()
