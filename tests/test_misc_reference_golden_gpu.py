"""GPU parity against outputs of further kernels of the reference's OWN compiled NVFP4 modules
(tests/golden/nvfp4_misc_reference_golden.npz, recorded by tests/golden/make_misc_reference_golden.py on a B200): the
16 x 16 weight quantiser, the SwiGLU element kernels, the three-stream gradient quantiser with stochastic rounding of
both axes, the rotary embedding of packed Q / K and its inverse, and the QKV projection with the rotary epilogue.
Bit-exact, no tolerance."""
import os

import numpy as np
import pytest
import torch

from tests.golden import make_misc_reference_golden as G
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16

pytestmark = pytest.mark.gpu

_PATH = os.path.join(os.path.dirname(__file__), "golden", "nvfp4_misc_reference_golden.npz")
GOLD = np.load(_PATH) if os.path.exists(_PATH) else None
needs_fixture = pytest.mark.skipif(GOLD is None, reason="fixture not recorded")
_u8 = lambda t: t.contiguous().view(torch.uint8).cpu().numpy()
_i16 = lambda t: t.view(torch.int16).cpu().numpy()


def _eq(key, got):
    want = GOLD[key]
    assert got.size == want.size, key
    bad = int((got.reshape(-1) != want.reshape(-1)).sum())
    assert bad == 0, f"{key}: {bad} of {got.size} values differ from the reference kernel's"


@needs_fixture
def test_split3_stochastic_both_axes():
    tkq = mod("tk_quant_v5")
    M, widths = G.SPLIT3
    ins = [to_dev_bf16(G.grads(M, n, 500 + i)) for i, n in enumerate(widths)]
    tkq.tk_set_sr_invocation_count(0)
    r = tkq.tk_group_quantize_dim1_split3_for_gemm(*ins, True, G.SEED, G.SUBSEQ, "both")
    torch.cuda.synchronize()
    assert tkq.tk_sr_invocation_count() == 3
    _eq("split3.row_fp4_full", _u8(r[5])); _eq("split3.row_sc_cat", _u8(r[6]))
    _eq("split3.col_fp4_full", _u8(r[7])); _eq("split3.col_sc_cat", _u8(r[8]))
    assert np.array_equal(r[2].cpu().numpy(), GOLD["split3.sg"]) and np.array_equal(r[12].cpu().numpy(), GOLD["split3.amax"])
    assert_status_ok()


@needs_fixture
def test_weight_2d_tiles():
    tkq = mod("tk_quant_v5")
    r = tkq.tk_quantize_weight_2d(to_dev_bf16(G.normal(256, 384, 510, 0.02)))
    torch.cuda.synchronize()
    for j in range(4):
        _eq(f"weight_2d.{j}", _u8(r[j]))
    assert r[4].item() == GOLD["weight_2d.sg"].reshape(-1)[0]
    assert_status_ok()


@needs_fixture
def test_swiglu_element_kernels():
    tkq = mod("tk_quant_v5")
    h1, h3, dh = to_dev_bf16(G.normal(256, 384, 520, 2.0)), to_dev_bf16(G.normal(256, 384, 521)), to_dev_bf16(G.grads(256, 384, 522))
    _eq("silu_mul", _i16(tkq.tk_silu_mul_split_bf16(h1, h3)))
    d1, d3 = tkq.tk_silu_deriv_split_bf16(dh, h3, h1)
    _eq("silu_deriv.dh1", _i16(d1)); _eq("silu_deriv.dh3", _i16(d3))
    assert_status_ok()


@needs_fixture
def test_rotary_embedding_of_packed_q_k_and_the_qkv_epilogue():
    gemm = mod("tk_gemm_c")
    R = G.ROPE
    cs = torch.from_numpy(G.rope_table(R["seq"], R["head"], 530)).cuda()
    q, k = to_dev_bf16(G.normal(R["M"], R["q_dim"], 531)), to_dev_bf16(G.normal(R["M"], R["kv_dim"], 532))
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    gemm.nvfp4_forward_rope_packed_qk(q, k, cs, R["seq"], R["head"], qo, ko)
    _eq("rope_fwd.q", _i16(qo)); _eq("rope_fwd.k", _i16(ko))
    gemm.nvfp4_inverse_rope_packed_qk(q, k, cs, R["seq"], R["head"], qo, ko)
    _eq("rope_inv.q", _i16(qo)); _eq("rope_inv.k", _i16(ko))
    # the packed operands the reference's quantiser made, through this library's GEMM with the rotary epilogue
    dev = "cuda"
    fp4, e4m3 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
    ld = lambda key, dt: torch.from_numpy(GOLD[key]).to(dev).view(dt)
    N = R["q_dim"] + 2 * R["kv_dim"]
    a, a_sc = ld("qkv_rope.a_fp4", fp4).view(R["M"], R["K"] // 2), ld("qkv_rope.a_sc", e4m3)
    b, b_sc = ld("qkv_rope.b_fp4", fp4).view(N, R["K"] // 2), ld("qkv_rope.b_sc", e4m3)
    a_sg = torch.from_numpy(GOLD["qkv_rope.a_sg"]).to(dev)
    b_sg = torch.from_numpy(GOLD["qkv_rope.b_sg"]).to(dev).expand(N // 256).contiguous()
    dq = torch.empty(R["M"], R["q_dim"], dtype=torch.bfloat16, device=dev)
    dk = torch.empty(R["M"], R["kv_dim"], dtype=torch.bfloat16, device=dev)
    dv = torch.empty(R["M"], R["kv_dim"], dtype=torch.bfloat16, device=dev)
    gemm.nvfp4_grouped_gemm_rope_packed_split(a, a_sc, a_sg, b, b_sc, b_sg, dq, dk, dv, cs, R["seq"], R["head"], R["head"])
    torch.cuda.synchronize()
    _eq("qkv_rope.q", _i16(dq)); _eq("qkv_rope.k", _i16(dk)); _eq("qkv_rope.v", _i16(dv))
    assert_status_ok()
