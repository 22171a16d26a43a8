"""GPU parity of the RMSNorm backward against the outputs of the reference's OWN kernels
(tests/golden/rmsnorm_bwd_kernels_golden.npz, recorded by tests/golden/make_rmsnorm_bwd_kernel_golden.py from the
reference's compiled ``_C`` module on a B200).  The three-stream form: d_sum, dx, the 256-row dgamma tiles and dgamma, bit
for bit.  The residual form: dx bit for bit; the reference adds its dgamma with atomics in no fixed order, so that
vector is compared to a few fp32 steps of the magnitude summed."""
import os

import numpy as np
import pytest
import torch

from tests.golden import make_rmsnorm_bwd_kernel_golden as G
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16

pytestmark = pytest.mark.gpu

_PATH = os.path.join(os.path.dirname(__file__), "golden", "rmsnorm_bwd_kernels_golden.npz")
GOLD = np.load(_PATH) if os.path.exists(_PATH) else None
_bits = lambda t: t.view(torch.int16).cpu().numpy()


def _same(key, array):
    """The fixture keeps a matrix as every eighth row (to say where a difference is) and the SHA-256 of all of it."""
    import hashlib
    a = np.ascontiguousarray(array)
    bad = int((a[::8] != GOLD[key + ".rows8"]).sum())
    assert bad == 0, f"{key}: {bad} values of the sampled rows differ from the reference kernel's"
    digest = np.frombuffer(hashlib.sha256(a.tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(digest, GOLD[key + ".sha256"]), f"{key}: the bytes outside the sampled rows differ"


@pytest.mark.skipif(GOLD is None, reason="fixture not recorded")
@pytest.mark.parametrize("idx", range(len(G.SUM3_SHAPES)))
def test_sum3_form_reproduces_the_reference_kernels_outputs(idx):
    gemm = mod("tk_gemm_c")
    M, K = G.SUM3_SHAPES[idx]
    d0, d1, d2, x, gamma = (to_dev_bf16(a) for a in G.make_inputs(M, K, 900 + idx))
    inv = torch.from_numpy(GOLD[f"sum3_{idx}.inv_rms"]).cuda()
    d_sum, dx = torch.empty_like(x), torch.empty_like(x)
    partials = torch.empty((M + 255) // 256, K, dtype=torch.float32, device="cuda")
    dgamma = torch.empty(K, dtype=torch.float32, device="cuda")
    gemm.sum3_rmsnorm_bwd_out(d0, d1, d2, x, gamma, inv, d_sum, dx, partials, dgamma)
    torch.cuda.synchronize()
    _same(f"sum3_{idx}.d_sum", _bits(d_sum))
    _same(f"sum3_{idx}.dx", _bits(dx))
    assert np.array_equal(partials.cpu().numpy(), GOLD[f"sum3_{idx}.partials"])
    assert np.array_equal(dgamma.cpu().numpy(), GOLD[f"sum3_{idx}.dgamma"])
    assert_status_ok()


@pytest.mark.skipif(GOLD is None, reason="fixture not recorded")
@pytest.mark.parametrize("idx", range(len(G.RESIDUAL_ROWS)))
def test_residual_form_reproduces_the_reference_kernels_dx(idx):
    gemm = mod("tk_gemm_c")
    M, K = G.RESIDUAL_ROWS[idx], 4096
    d0, d1, _, x, gamma = (to_dev_bf16(a) for a in G.make_inputs(M, K, 950 + idx))
    inv = torch.from_numpy(GOLD[f"residual_{idx}.inv_rms"]).cuda()
    dx = torch.empty_like(x)
    dgamma = torch.empty(K, dtype=torch.float32, device="cuda")
    gemm.rmsnorm_bwd_residual_out(d0, x, gamma, inv, d1, dx, dgamma)
    torch.cuda.synchronize()
    _same(f"residual_{idx}.dx", _bits(dx))
    want = GOLD[f"residual_{idx}.dgamma"]
    scale = float(np.abs(want).max())
    assert np.abs(dgamma.cpu().numpy() - want).max() <= 1e-5 * scale
    assert_status_ok()
