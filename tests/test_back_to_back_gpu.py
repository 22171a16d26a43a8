"""Calls of the fused RMSNorm + NVFP4 producer issued back to back on one stream.  The statistics kernel of a call
may start while the quantiser of the previous call still runs (programmatic dependent launch): it stages gamma and
prefetches its input, and has to hold every write until that quantiser has ended.  Here consecutive calls alternate
between two inputs, SHARE the inv_rms and tensor-scale buffers and write separate operand buffers, at the benchmark
size, so that an early write of inv_rms or of the partial maxima would corrupt the previous call's operands."""
import importlib

import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture
def early_reads(request):
    """Sets the library's early-reads switch for one test and restores it."""
    lib = importlib.import_module("mfu-fp4-training_b200._lib").load()
    before = lib.fp4b200_set_pdl_early_reads(int(request.param))
    yield bool(request.param)
    lib.fp4b200_set_pdl_early_reads(before)


@pytest.mark.parametrize("early_reads", [0, 1], indirect=True)
@pytest.mark.parametrize("shape", [(16384, 4096), (2048, 1024)])
def test_back_to_back_calls_sharing_inv_rms_do_not_disturb_each_other(shape, early_reads):
    lib = importlib.import_module("mfu-fp4-training_b200._lib")
    M, K = shape
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    xs = [(torch.randn((M, K), generator=g, device=dev) * s).to(torch.bfloat16) for s in (1.0, 3.0)]
    xs[1][:, 7] *= 20.0                                     # the two inputs differ in tensor maximum and row norms
    gamma = to_dev_bf16(o.make_gamma(K, seed=3))
    inv_rms = torch.empty(M, dtype=torch.float32, device=dev)
    amax_sg = torch.empty(2, dtype=torch.float32, device=dev)
    u8 = dict(dtype=torch.uint8, device=dev)
    n_calls = 12
    outs = [(torch.empty((M, K // 2), **u8), torch.empty((M // 128, K // 64, 512), **u8),
             torch.empty((K, M // 2), **u8), torch.empty((K // 128, M // 64, 512), **u8)) for _ in range(n_calls)]
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    for i, (rf, rs, cf, cs) in enumerate(outs):
        lib.call("fp4b200_nvfp4_fused_norm_quantize", xs[i % 2].data_ptr(), gamma.data_ptr(), 1e-5, M, K, inv_rms.data_ptr(), 1,
                 1, rf.data_ptr(), rs.data_ptr(), cf.data_ptr(), cs.data_ptr(), amax_sg.data_ptr(), stream)
    torch.cuda.synchronize()
    # calls 0 and 1 against single calls made in isolation
    for k in range(2):
        alone = [torch.empty_like(t) for t in outs[k]]
        lib.call("fp4b200_nvfp4_fused_norm_quantize", xs[k].data_ptr(), gamma.data_ptr(), 1e-5, M, K, inv_rms.data_ptr(), 1, 1,
                 alone[0].data_ptr(), alone[1].data_ptr(), alone[2].data_ptr(), alone[3].data_ptr(), amax_sg.data_ptr(), stream)
        torch.cuda.synchronize()
        for i in range(k, n_calls, 2):
            for got, want in zip(outs[i], alone):
                assert torch.equal(got, want), f"call {i} differs from the same call made alone"
    assert not torch.equal(outs[0][0], outs[1][0])
    if M <= 2048:   # small case: the isolated result is the oracle's
        x = xs[1].float().cpu().numpy()
        inv = o.rmsnorm_inv_rms(x, 1e-5)
        ref = o.nvfp4_quantize_for_gemm(o.rmsnorm_apply(x, inv_rms.cpu().numpy(), gamma.float().cpu().numpy()), True, True)
        assert np.array_equal(outs[1][0].cpu().numpy(), ref["row_fp4"]) and np.array_equal(outs[1][2].cpu().numpy(), ref["col_fp4"])
        assert np.abs(inv_rms.cpu().numpy() / inv - 1).max() < 2e-6
    assert_status_ok()


@pytest.mark.parametrize("shape", [(16384, 4096), (512, 1024)])
def test_input_rewritten_by_the_previous_kernel_is_read_after_it(shape):
    """The usual call pattern of a training step: the kernel launched just before the producer (here a torch copy,
    in a model the residual add or a GEMM epilogue) writes the very buffer the producer reads.  The first-pass
    kernels are programmatic dependents, so they must not read x or gamma before that kernel's writes are visible
    (the library's default).  Every call is compared with the same call made alone on settled memory; both the fused
    RMSNorm producer and the plain quantiser (tensor-maximum kernel in front) are covered."""
    lib = importlib.import_module("mfu-fp4-training_b200._lib")
    M, K = shape
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(11)
    srcs = [(torch.randn((M, K), generator=g, device=dev) * s).to(torch.bfloat16) for s in (1.0, 5.0, 0.25)]
    gammas = [to_dev_bf16(o.make_gamma(K, seed=s)) for s in (3, 4, 5)]
    x = torch.empty((M, K), dtype=torch.bfloat16, device=dev)        # the one buffer every call reads
    gamma = torch.empty(K, dtype=torch.bfloat16, device=dev)
    inv_rms = torch.empty(M, dtype=torch.float32, device=dev)
    amax_sg = torch.empty(2, dtype=torch.float32, device=dev)
    u8 = dict(dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def outs():
        return (torch.empty((M, K // 2), **u8), torch.empty((M // 128, K // 64, 512), **u8),
                torch.empty((K, M // 2), **u8), torch.empty((K // 128, M // 64, 512), **u8))

    def fused(o4):
        lib.call("fp4b200_nvfp4_fused_norm_quantize", x.data_ptr(), gamma.data_ptr(), 1e-5, M, K, inv_rms.data_ptr(), 1, 1,
                 o4[0].data_ptr(), o4[1].data_ptr(), o4[2].data_ptr(), o4[3].data_ptr(), amax_sg.data_ptr(), stream)

    def plain(o4):
        lib.call("fp4b200_nvfp4_quantize_for_gemm", x.data_ptr(), M, K, 1, 1, o4[0].data_ptr(), o4[1].data_ptr(),
                 o4[2].data_ptr(), o4[3].data_ptr(), amax_sg.data_ptr(), stream)

    for call in (fused, plain):
        n_calls = 9
        got = [outs() for _ in range(n_calls)]
        torch.cuda.synchronize()
        for i in range(n_calls):
            x.copy_(srcs[i % 3])            # the kernel right in front of the producer writes its input ...
            gamma.copy_(gammas[i % 3])      # ... and its weight
            call(got[i])
        torch.cuda.synchronize()
        for k in range(3):
            x.copy_(srcs[k])
            gamma.copy_(gammas[k])
            torch.cuda.synchronize()
            alone = outs()
            call(alone)
            torch.cuda.synchronize()
            for i in range(k, n_calls, 3):
                for a, b in zip(got[i], alone):
                    assert torch.equal(a, b), f"{call.__name__}: call {i} read its input before the copy in front of it had landed"
    assert_status_ok()
