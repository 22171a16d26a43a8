"""GPU: the entry point that allocates nothing (fp4b200_nvfp4_fused_norm_quantize_noalloc).

Some callers of this library cannot allocate device memory when they need the fused producer:
code that runs under a memory budget that is already fully handed out, or in a thread that must
not touch the allocator.  For them the library keeps the producer's scratch (inverse RMS per row, tensor amax)
in a fixed device array of its own.  This test calls that entry point through the C ABI twice in a
row, with different inputs, and checks every output byte against the ordinary entry point, which
uses caller-provided buffers: the second call must not see anything left over from the first.
It is collected last so that a run stopping at the first failure has already run the other tests.
"""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16

pytestmark = pytest.mark.gpu


def _run_both(lib, x, g, eps):
    M, K = x.shape
    dev = x.device
    u8 = dict(dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def bufs():
        return (torch.full((M, K // 2), 0xAA, **u8), torch.full((M * K // 16,), 0xAA, **u8),
                torch.full((K, M // 2), 0xAA, **u8), torch.full((M * K // 16,), 0xAA, **u8))

    a = bufs()
    sg_a = torch.zeros(1, dtype=torch.float32, device=dev)
    lib.call("fp4b200_nvfp4_fused_norm_quantize_noalloc", x.data_ptr(), g.data_ptr(), eps, M, K,
             a[0].data_ptr(), a[1].data_ptr(), a[2].data_ptr(), a[3].data_ptr(), sg_a.data_ptr(), stream)
    b = bufs()
    inv = torch.empty(M, dtype=torch.float32, device=dev)
    amax_sg = torch.empty(2, dtype=torch.float32, device=dev)
    lib.call("fp4b200_nvfp4_fused_norm_quantize", x.data_ptr(), g.data_ptr(), eps, M, K, inv.data_ptr(), 1, 1,
             b[0].data_ptr(), b[1].data_ptr(), b[2].data_ptr(), b[3].data_ptr(), amax_sg.data_ptr(), stream)
    torch.cuda.synchronize()
    for got, want, name in zip(a, b, ("row codes", "row scales", "column codes", "column scales")):
        assert torch.equal(got, want), f"{name} differ from the allocating entry point"
    assert sg_a.item() == amax_sg[1].item()


def test_noalloc_matches_allocating_entry_point_twice():
    lib = mod("_lib")
    # first call: a large-amplitude tensor; second call: a smaller one with a smaller amax and
    # fewer rows, so stale scratch from the first call would change the result
    x1 = to_dev_bf16(o.make_activations(512, 1024, seed=101, scale=4.0))
    g1 = to_dev_bf16(o.make_gamma(1024, seed=102))
    _run_both(lib, x1, g1, 1e-5)
    x2 = to_dev_bf16(o.make_activations(256, 512, seed=103, scale=0.05, outlier_frac=0))
    g2 = to_dev_bf16(o.make_gamma(512, seed=104))
    _run_both(lib, x2, g2, 1e-5)
    assert_status_ok()


def test_noalloc_against_the_oracle():
    """The same entry point against the CPU oracle alone, so that its check does not lean on another entry point of
    this library.  The oracle's inverse RMS comes from a float32 tree and a correctly rounded reciprocal square root,
    the GPU's from its own `rsqrtf` (<= 2e-6 relative apart), and this entry point does not hand its inverse RMS out;
    a normalised value that sits on a bf16 rounding boundary may therefore land one code apart: at most 1 byte in
    1000 may differ, and the tensor scale to 1 part in 1e5."""
    lib = mod("_lib")
    M, K = 256, 512
    x = o.make_activations(M, K, seed=211)
    gamma = o.make_gamma(K, seed=212)
    xd, gd = to_dev_bf16(x), to_dev_bf16(gamma)
    u8 = dict(dtype=torch.uint8, device="cuda")
    out = (torch.empty((M, K // 2), **u8), torch.empty((M * K // 16,), **u8), torch.empty((K, M // 2), **u8),
           torch.empty((M * K // 16,), **u8))
    sg = torch.zeros(1, dtype=torch.float32, device="cuda")
    for _ in range(2):
        lib.call("fp4b200_nvfp4_fused_norm_quantize_noalloc", xd.data_ptr(), gd.data_ptr(), 1e-5, M, K, out[0].data_ptr(),
                 out[1].data_ptr(), out[2].data_ptr(), out[3].data_ptr(), sg.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    inv = o.rmsnorm_inv_rms(x, 1e-5)
    ref = o.nvfp4_quantize_for_gemm(o.rmsnorm_apply(x, inv, o.bf16_round(gamma)), True, True)
    assert abs(sg.item() / ref["sg"] - 1.0) < 1e-5
    for got, key in zip(out, ("row_fp4", "row_sc", "col_fp4", "col_sc")):
        got = got.cpu().numpy().reshape(-1)
        want = np.asarray(ref[key]).reshape(-1)
        assert got.size == want.size
        assert (got != want).mean() <= 1e-3, f"{key}: {(got != want).mean():.5f} of the bytes differ from the oracle"
    assert_status_ok()


def test_noalloc_rejects_too_many_rows():
    lib = mod("_lib")
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        lib.call("fp4b200_nvfp4_fused_norm_quantize_noalloc", x.data_ptr(), x.data_ptr(), 1e-5, 65536 + 128, 128,
                 x.data_ptr(), x.data_ptr(), None, None, x.data_ptr(), None)
