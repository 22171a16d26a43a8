"""The allocate-once / launch-many pairs and the other entry points inside CUDA graph capture: a captured call,
replayed on new input data, gives the same bytes as an eager call on that data."""
import numpy as np
import pytest
import torch

from oracle import fp4_oracle as o
from tests.gpu_util import assert_status_ok, mod, to_dev_bf16

pytestmark = pytest.mark.gpu


def _capture(fn, warm):
    """Runs `warm` once on a side stream (the library creates its per-stream scratch on a stream's first call),
    captures `fn` on that stream and returns the graph."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        warm()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        fn()
    return g


def test_v4_quantize_pair_in_a_graph():
    tkq = mod("tk_quant_v5")
    M, K = 512, 1024
    x = to_dev_bf16(o.make_activations(M, K, seed=1))
    bufs = tkq.tk_v4_quantize_for_gemm_alloc(M, K, True, x.device)
    res = {}

    def launch():
        res["out"] = tkq.tk_v4_quantize_for_gemm_launch(x, True, True, *bufs)

    g = _capture(launch, launch)
    x2 = o.make_activations(M, K, seed=2)
    x.copy_(to_dev_bf16(x2))
    g.replay()
    torch.cuda.synchronize()
    ref = o.nvfp4_quantize_for_gemm(x2, True, True)
    out = res["out"]
    for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]):
        assert np.array_equal(out[i].view(torch.uint8).cpu().numpy().reshape(ref[k].shape), ref[k]), k
    assert out[4].item() == ref["sg"] and bufs[4][0].item() == ref["amax"]
    assert_status_ok()


def test_silu_deriv_split_pair_in_a_graph_equals_the_allocating_call():
    tkq = mod("tk_quant_v5")
    M, H = 256, 512
    rng = np.random.default_rng(5)
    mk = lambda s: to_dev_bf16(o.bf16_round((s * rng.standard_normal((M, H))).astype(np.float32)))
    dh, h3, h1 = mk(1e-3), mk(1.0), mk(2.0)
    bufs = tkq.tk_silu_deriv_quantize_split_for_gemm_alloc(M, H, dh.device)
    res = {}

    def launch():
        res["out"] = tkq.tk_silu_deriv_quantize_split_for_gemm_launch(dh, h3, h1, *bufs)

    g = _capture(launch, launch)
    for t, s in ((dh, 2e-3), (h3, 0.5), (h1, 1.5)):
        t.copy_(mk(s))
    g.replay()
    torch.cuda.synchronize()
    eager = tkq.tk_silu_deriv_quantize_split_for_gemm(dh, h3, h1)
    torch.cuda.synchronize()
    out = res["out"]
    assert len(out) == 12
    for i in (0, 1, 2, 3, 6, 7, 8, 9):
        assert torch.equal(out[i].view(torch.uint8), eager[i].view(torch.uint8)), i
    assert torch.equal(out[4], eager[4]) and torch.equal(out[10], eager[10])          # sg of dh1 / dh3
    assert torch.equal(bufs[10], eager[12])                                           # the two tensor maxima
    assert torch.equal(bufs[12], eager[14]) and torch.equal(bufs[13], eager[15])     # dh1, dh3
    assert out[5].item() == 0.0
    assert_status_ok()


def test_fused_norm_quantize_and_rmsnorm_backward_in_a_graph():
    """The fused producer (two launches, the second programmatically dependent on the first) and the RMSNorm
    backward (cooperative launch) are captured with their allocating mirrors: torch's graph pool serves them."""
    tkq, gemm = mod("tk_quant_v5"), mod("tk_gemm_c")
    M, K = 512, 1024
    x = to_dev_bf16(o.make_activations(M, K, seed=3))
    g_w = to_dev_bf16(o.make_gamma(K, seed=4))
    d = [to_dev_bf16(o.bf16_round((1e-3 * np.random.default_rng(6 + i).standard_normal((M, K))).astype(np.float32)))
         for i in range(3)]
    d_sum, dx = torch.empty_like(x), torch.empty_like(x)
    partials = torch.empty((M // 256, K), dtype=torch.float32, device="cuda")
    dgamma = torch.empty(K, dtype=torch.float32, device="cuda")
    res = {}

    def step():
        res["q"] = tkq.tk_fused_norm_quantize(x, g_w, 1e-5, False, True)
        gemm.sum3_rmsnorm_bwd_out(d[0], d[1], d[2], x, g_w, res["q"][5], d_sum, dx, partials, dgamma)

    g = _capture(step, step)
    x2 = o.make_activations(M, K, seed=9)
    x.copy_(to_dev_bf16(x2))
    g.replay()
    torch.cuda.synchronize()
    q = [t.clone() for t in res["q"][:6]]
    dx_g, dg_g = dx.clone(), dgamma.clone()
    eager = tkq.tk_fused_norm_quantize(x, g_w, 1e-5, False, True)
    gemm.sum3_rmsnorm_bwd_out(d[0], d[1], d[2], x, g_w, eager[5], d_sum, dx, partials, dgamma)
    torch.cuda.synchronize()
    for i in range(4):
        assert torch.equal(q[i].view(torch.uint8), eager[i].view(torch.uint8)), i
    assert torch.equal(q[5], eager[5]) and torch.equal(dx_g, dx) and torch.equal(dg_g, dgamma)
    assert_status_ok()


def test_captured_stochastic_rounding_draws_anew_on_every_replay():
    """The NVFP4 stochastic quantisers number their launches on the device (a one-thread kernel advances the counter
    and hands the launch its key and offset through device memory, as the reference does), so a captured call
    reserves a new launch number on every replay: replay k gives the bytes of the eager call made with the counter
    at the value replay k found.  The MXFP4 forms still count on the host and refuse to be captured."""
    tkq, mxq = mod("tk_quant_v5"), mod("mxfp4_quant_v4")
    x = (1e-3 * torch.randn(256, 256, device="cuda")).to(torch.bfloat16)
    args = (x, True, False, True, False, "none", False, 77, 5, 448.0, "both")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        tkq.tk_quantize_for_gemm_opt(*args)                 # the stream's first call (per-stream scratch) outside capture
    side.synchronize()
    tkq.tk_set_sr_invocation_count(40)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        with pytest.raises(RuntimeError, match="graph"):
            mxq.mxfp4_quantize_row_and_col_opt(x, 1, True, False, 1, 0)
        out = tkq.tk_quantize_for_gemm_opt(*args)
    assert tkq.tk_sr_invocation_count() == 40               # capturing launches nothing
    replays = []
    for _ in range(3):
        g.replay()
        torch.cuda.synchronize()
        replays.append([t.view(torch.uint8).clone() for t in out[:4]])
    assert tkq.tk_sr_invocation_count() == 43
    assert not torch.equal(replays[0][0], replays[1][0]) and not torch.equal(replays[1][2], replays[2][2])
    for k in range(3):
        tkq.tk_set_sr_invocation_count(40 + k)
        eager = tkq.tk_quantize_for_gemm_opt(*args)
        for a, b in zip(replays[k], eager[:4]):
            assert torch.equal(a, b.view(torch.uint8))
    assert_status_ok()


def test_a_producers_own_counter_feeds_the_quantiser_and_advances_in_captured_replays():
    """producer_sr_state: the stochastic quantisers take key and base from a producer's persistent {seed, next
    subsequence} row (a LocalCTASRState table on the device) and advance the row by 2**32 per launch on their own
    stream; the device-wide counter is not touched.  The bytes are those of the explicit call with that seed and
    subsequence at launch number 0.  Captured, every replay advances the live row; what warm-up and capture reserved
    is rolled back by preserve_during_cuda_graph_capture."""
    tkq, srs = mod("tk_quant_v5"), mod("localcta_sr_state")
    keys = [srs.ffn_w2_grad_key("layers.0.ffn"), srs.qkv_grad_key("layers.0.attn:qkv")]
    table = srs.LocalCTASRState(keys, device="cuda", user_seed=(1 << 64) - 2, user_subsequence_base=9 << 32,
                                training_steps=4, gradient_accumulation_steps=1)
    x = (1e-3 * torch.randn(256, 256, device="cuda")).to(torch.bfloat16)
    U64 = (1 << 64) - 1

    def call(seed=0, sub=0):
        return tkq.tk_quantize_for_gemm_opt(x, True, False, True, False, "none", False, seed, sub, 448.0, "both")

    def explicit(row):
        tkq.tk_set_sr_invocation_count(0)
        return [t.view(torch.uint8).clone() for t in call(int(row[0]) & U64, int(row[1]) & U64)[:4]]

    tkq.tk_set_sr_invocation_count(11)
    row = table.get(keys[1], x.device)
    other = table.get(keys[0]).clone()
    before = row.clone()
    with tkq.producer_sr_state(row):
        got = [t.view(torch.uint8).clone() for t in call(123, 456)]     # seed / subsequence arguments are ignored
        launches = (int(row[1]) - int(before[1])) >> 32
        assert launches >= 1 and int(row[0]) == int(before[0])
        with tkq.producer_sr_state(None):                               # None: the device-wide numbering again
            call()
    assert tkq.tk_sr_invocation_count() == 11 + launches                # only the inner, unbound call counted there
    assert torch.equal(table.get(keys[0]), other)
    for a, b in zip(got, explicit(before)):
        assert torch.equal(a, b)
    with pytest.raises(RuntimeError, match="contiguous CUDA int64 tensor with two elements"):
        with tkq.producer_sr_state(torch.zeros(2, dtype=torch.int64)):
            pass

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    start = row.clone()
    with table.preserve_during_cuda_graph_capture([keys[1]]):
        with torch.cuda.stream(side), tkq.producer_sr_state(row):
            call()                                                       # warm-up on the capture stream
        side.synchronize()
        with torch.cuda.graph(g, stream=side), tkq.producer_sr_state(row):
            out = call()
    assert torch.equal(row, start)                                       # warm-up and capture left no trace
    replays = []
    for _ in range(2):
        g.replay()
        torch.cuda.synchronize()
        replays.append([t.view(torch.uint8).clone() for t in out[:4]])
    assert (int(row[1]) - int(start[1])) >> 32 == 2 * launches
    assert not torch.equal(replays[0][0], replays[1][0])
    for k in range(2):
        at = start.clone()
        at[1] += k * launches * (1 << 32)
        for a, b in zip(replays[k], explicit(at)):
            assert torch.equal(a, b)
    sd = table.state_dict()
    assert sd["states"][0, table.logical_keys.index(keys[1])].tolist() == row.tolist()
    assert_status_ok()


def test_split2_opt_pair_captures_and_equals_its_parts():
    """tk_silu_deriv_quantize_split_for_gemm_opt_alloc / _launch: buffers once, launch captured, replayed on new data.
    Each of dh1 / dh3 equals the single-launch quantiser (row operand transformed, both passes one random stream) on
    the bf16 intermediate at the launch number the pair reserved: one number for both, as in the reference's kernel
    for this pair."""
    tkq = mod("tk_quant_v5")
    M, H = 256, 384
    def inputs(seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        return ((1e-3 * torch.randn(M, H, device="cuda", generator=g)).to(torch.bfloat16),
                torch.randn(M, H, device="cuda", generator=g).to(torch.bfloat16),
                torch.randn(M, H, device="cuda", generator=g).to(torch.bfloat16))
    dh, h3, h1 = inputs(1)
    bufs = tkq.tk_silu_deriv_quantize_split_for_gemm_opt_alloc(M, H, dh.device)
    def launch():
        return tkq.tk_silu_deriv_quantize_split_for_gemm_opt_launch(dh, h3, h1, True, False, True, True, "row", False, 9, 2,
                                                                    *bufs, "both")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch()
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        out = launch()
    for seed, count in ((2, 11), (3, 12)):
        a, b, c = inputs(seed)
        dh.copy_(a); h3.copy_(b); h1.copy_(c)
        tkq.tk_set_sr_invocation_count(count)
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        assert tkq.tk_sr_invocation_count() == count + 1    # one number for the whole pair
        d1, d3 = tkq.tk_silu_deriv_split_bf16(dh, h3, h1)
        for t, o in ((d1, out[0:6]), (d3, out[6:12])):
            row_amax = tkq._amax_rht(t, True, False, 0, 0)
            plain = tkq._amax_plain(t)
            state = torch.tensor([9, 2 + (count << 32)], dtype=torch.int64, device=t.device)
            ref = tkq.tk_quantize_transpose(t, row_amax, plain, True, True, False, True, True, False, True, state)
            for got, want in zip(o[:4], ref):
                assert torch.equal(got.view(torch.uint8).reshape(-1), want.view(torch.uint8).reshape(-1))
            assert float(o[4]) == float(row_amax[1]) and float(o[5]) == float(plain[1])
    with pytest.raises(RuntimeError, match="one axis"):
        tkq.tk_silu_deriv_quantize_split_for_gemm_opt_launch(dh, h3, h1, True, False, True, False, "row", False, 9, 2, *bufs, "row")
    assert_status_ok()
