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


@pytest.mark.parametrize("shape", [(16384, 4096), (2048, 1024)])
def test_back_to_back_calls_sharing_inv_rms_do_not_disturb_each_other(shape):
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
