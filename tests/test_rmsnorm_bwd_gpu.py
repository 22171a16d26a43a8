"""GPU parity of the RMSNorm backward entry points (the step right behind the dgrad GEMMs): every output
bit-exact against the oracle's restatement of the reference kernels at sizes the oracle finishes in seconds;
at the benchmark size sampled rows and tiles bit-exact, the whole result against an fp32 torch formula, and
determinism."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16

pytestmark = pytest.mark.gpu


def _bf16(a):
    return o.bf16_round(np.asarray(a, dtype=np.float32))


def _inputs(M, K, seed):
    rng = np.random.default_rng(seed)
    d = [_bf16(1e-3 * rng.standard_normal((M, K))) for _ in range(3)]
    x = o.make_activations(M, K, seed=seed + 1)
    g = o.make_gamma(K, seed=seed + 2)
    inv = o.rmsnorm_inv_rms(x, 1e-5)
    return d, x, g, inv


def _f32(t):
    return t.float().cpu().numpy()


@pytest.mark.parametrize("dgamma_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 256), (300, 1024), (513, 4096), (1024, 768), (260, 8192), (130, 6144)])
def test_sum3_rmsnorm_bwd_bit_exact(shape, dgamma_dtype):
    gemm = mod("tk_gemm_c")
    M, K = shape
    d, x, g, inv = _inputs(M, K, seed=M + K)
    dev = [to_dev_bf16(a) for a in d]
    xd, gd = to_dev_bf16(x), to_dev_bf16(g)
    invd = torch.from_numpy(inv).cuda()
    d_sum = torch.empty_like(xd)
    dx = torch.empty_like(xd)
    tiles = (M + 255) // 256
    partials = torch.full((tiles, K), float("nan"), dtype=torch.float32, device="cuda")
    dgamma = torch.empty(K, dtype=dgamma_dtype, device="cuda")
    gemm.sum3_rmsnorm_bwd_out(dev[0], dev[1], dev[2], xd, gd, invd, d_sum, dx, partials, dgamma)
    torch.cuda.synchronize()
    assert_status_ok()
    ref = o.sum3_rmsnorm_bwd(d[0], d[1], d[2], x, g, inv)
    assert np.array_equal(_f32(d_sum), ref["d_sum"])
    assert np.array_equal(_f32(dx), ref["grad_input"])
    assert np.array_equal(partials.cpu().numpy(), ref["dgamma_partials"])
    want = ref["dgamma"] if dgamma_dtype == torch.float32 else o.bf16_round(ref["dgamma"])
    assert np.array_equal(_f32(dgamma), want)


@pytest.mark.parametrize("M", [1, 260, 1024])
def test_rmsnorm_bwd_residual(M):
    gemm = mod("tk_gemm_c")
    K = 4096
    d, x, g, inv = _inputs(M, K, seed=M + 5)
    dy, res = d[0], _bf16(10 * d[1])
    dyd, resd, xd, gd = to_dev_bf16(dy), to_dev_bf16(res), to_dev_bf16(x), to_dev_bf16(g)
    invd = torch.from_numpy(inv).cuda()
    dx = torch.empty_like(xd)
    dgamma = torch.empty(K, dtype=torch.float32, device="cuda")
    gemm.rmsnorm_bwd_residual_out(dyd, xd, gd, invd, resd, dx, dgamma)
    dx2 = torch.empty_like(xd)
    dgamma2 = torch.empty_like(dgamma)
    gemm.rmsnorm_bwd_residual_out(dyd, xd, gd, invd, resd, dx2, dgamma2)
    torch.cuda.synchronize()
    assert_status_ok()
    ref = o.rmsnorm_bwd_residual(dy, x, g, inv, res)
    assert np.array_equal(_f32(dx), ref["grad_input"])
    # the reference's atomics fix no order: any fp32 summation order of the same terms is admissible
    got = dgamma.cpu().numpy().astype(np.float64)
    scale = np.abs(ref["dgamma"]).max() + 1e-30
    assert np.abs(got - ref["dgamma"]).max() <= 1e-5 * scale * max(1.0, np.sqrt(M))
    assert torch.equal(dx, dx2) and torch.equal(dgamma, dgamma2)   # reproducible, unlike the atomics


def test_rmsnorm_bwd_rejects_bad_arguments():
    gemm = mod("tk_gemm_c")
    M, K = 256, 512
    z = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
    g = torch.ones(K, dtype=torch.bfloat16, device="cuda")
    inv = torch.ones(M, dtype=torch.float32, device="cuda")
    part = torch.empty((1, K), dtype=torch.float32, device="cuda")
    dg = torch.empty(K, dtype=torch.float32, device="cuda")
    outs = [torch.empty_like(z) for _ in range(2)]
    with pytest.raises(RuntimeError):   # d_sum aliases an input
        gemm.sum3_rmsnorm_bwd_out(z, z.clone(), z.clone(), z.clone(), g, inv, z, outs[1], part, dg)
    with pytest.raises(RuntimeError):   # wrong tile count
        gemm.sum3_rmsnorm_bwd_out(z, z.clone(), z.clone(), z.clone(), g, inv, outs[0], outs[1],
                                  torch.empty((2, K), dtype=torch.float32, device="cuda"), dg)
    with pytest.raises(RuntimeError):   # K = 512 is not the residual form's 4096
        gemm.rmsnorm_bwd_residual_out(z, z.clone(), g, inv, z.clone(), outs[0], dg)
    z3 = torch.zeros((M, 384), dtype=torch.bfloat16, device="cuda")   # K not a multiple of 256
    with pytest.raises(RuntimeError):
        gemm.sum3_rmsnorm_bwd_out(z3, z3.clone(), z3.clone(), z3.clone(), g[:384].contiguous(), inv, torch.empty_like(z3),
                                  torch.empty_like(z3), torch.empty((1, 384), dtype=torch.float32, device="cuda"),
                                  torch.empty(384, dtype=torch.float32, device="cuda"))
    assert_status_ok()


def test_sum3_rmsnorm_bwd_full_size():
    """16384 x 4096 (the backward configuration's dY): sampled rows and one row tile bit-exact against the oracle,
    everything against the fp32 formula, and two runs bit-identical."""
    gemm = mod("tk_gemm_c")
    M, K = 16384, 4096
    gen = torch.Generator(device="cuda").manual_seed(3)
    dev = [(1e-3 * torch.randn((M, K), generator=gen, device="cuda")).to(torch.bfloat16) for _ in range(3)]
    xd = torch.randn((M, K), generator=gen, device="cuda").to(torch.bfloat16)
    gd = (1 + 0.1 * torch.randn(K, generator=gen, device="cuda")).to(torch.bfloat16)
    invd = torch.rsqrt(xd.float().pow(2).mean(dim=1) + 1e-5)
    outs = []
    for _ in range(2):
        d_sum, dx = torch.empty_like(xd), torch.empty_like(xd)
        partials = torch.empty((M // 256, K), dtype=torch.float32, device="cuda")
        dgamma = torch.empty(K, dtype=torch.float32, device="cuda")
        gemm.sum3_rmsnorm_bwd_out(dev[0], dev[1], dev[2], xd, gd, invd, d_sum, dx, partials, dgamma)
        outs.append((d_sum, dx, partials, dgamma))
    torch.cuda.synchronize()
    assert_status_ok()
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    d_sum, dx, partials, dgamma = outs[0]
    assert torch.equal(d_sum, (dev[0] + dev[1]) + dev[2])
    # fp32 formula over the whole tensor
    dyf, xh = d_sum.float(), xd.float() * invd[:, None]
    mean = (dyf * xh * gd.float()).sum(dim=1, keepdim=True) / K
    want = invd[:, None] * (dyf * gd.float() - xh * mean)
    err = (dx.float() - want).abs().max().item() / want.abs().max().item()
    assert err < 1e-2
    dg_ref = (dyf.double() * xh.double()).sum(dim=0)
    assert (dgamma.double() - dg_ref).abs().max().item() <= 1e-4 * dg_ref.abs().max().item()
    # sampled rows, and the last row tile, bit-exact
    rows = np.array([0, 1, 255, 256, 8191, 16383])
    ridx = torch.from_numpy(rows).cuda()
    g_np, inv_np = _f32(gd), invd.cpu().numpy()
    ref = o.sum3_rmsnorm_bwd(*[_f32(t[ridx]) for t in dev], _f32(xd[ridx]), g_np, inv_np[rows])
    assert np.array_equal(_f32(dx[ridx]), ref["grad_input"])
    t0 = M - 256
    tile = o.rmsnorm_bwd_dgamma_tiles(_f32(d_sum[t0:]), _f32(xd[t0:]), inv_np[t0:])[0]
    assert np.array_equal(partials[-1].cpu().numpy(), tile[0])
    assert np.array_equal(dgamma.cpu().numpy(), _sum_tiles(partials.cpu().numpy()))


def _sum_tiles(p):
    acc = np.zeros(p.shape[1], dtype=np.float32)
    for t in range(p.shape[0]):
        acc = (acc + p[t]).astype(np.float32)
    return acc
