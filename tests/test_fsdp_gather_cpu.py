"""CPU, world_size 2 over gloo: the packed-weight all-gather reproduces, byte for byte, the
operands obtained by quantising the full weight — exchange logic only, with the oracle standing in
for the CUDA quantiser (which needs a GPU)."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_nvfp4(w_shard, amax, encode_centric, want_col):
    from oracle import fp4_oracle as o
    r = o.nvfp4_quantize_for_gemm(w_shard.float().numpy(), want_col, encode_centric, amax=amax.item())
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    return t(r["row_fp4"]), t(r["row_sc"]), t(r["col_fp4"]) if want_col else None, t(r["col_sc"]) if want_col else None


def _oracle_mxfp4(w_shard, mode, want_col):
    from oracle import fp4_oracle as o
    r = o.mxfp4_quantize_row_and_col(w_shard.float().numpy(), mode)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    return t(r["row_fp4"]), t(r["row_sc"]), t(r["col_fp4"]), t(r["col_sc"])


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import fp4_oracle as o
        fsdp = importlib.import_module("mfu-fp4-training_b200.fsdp_weights")
        N, K = 512, 256
        w = o.bf16_round((0.02 * np.random.default_rng(5).standard_normal((N, K))).astype(np.float32))
        w[300, 17] = 0.5      # the tensor amax lives in rank 1's shard only
        w = o.bf16_round(w)
        shard = torch.from_numpy(w[rank * N // world:(rank + 1) * N // world]).to(torch.bfloat16).contiguous()
        out = fsdp.all_gather_nvfp4_weight(shard, None, True, True, quantize_shard=_oracle_nvfp4)
        ref = o.nvfp4_quantize_for_gemm(w, True, True)
        ok = all(np.array_equal(out[i].numpy().reshape(ref[k].shape), ref[k])
                 for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]))
        ok = ok and out[4].item() == ref["sg"]
        out = fsdp.all_gather_mxfp4_weight(shard, None, True, 1, quantize_shard=_oracle_mxfp4)
        ref = o.mxfp4_quantize_row_and_col(w, 1)
        ok = ok and all(np.array_equal(out[i].numpy().reshape(ref[k].shape), ref[k])
                        for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]))
        # a layer's weights at once: one amax all-reduce over the stacked maxima, one group of all-gathers
        w2 = o.bf16_round((0.03 * np.random.default_rng(6).standard_normal((256, 384))).astype(np.float32))
        w2[5, 5] = -0.75      # this one's tensor amax lives in rank 0's shard
        w2 = o.bf16_round(w2)
        shard2 = torch.from_numpy(w2[rank * 256 // world:(rank + 1) * 256 // world]).to(torch.bfloat16).contiguous()
        for want_col in (True, False):
            outs = fsdp.all_gather_nvfp4_weights([shard, shard2], None, want_col, True, quantize_shard=_oracle_nvfp4)
            for got, full in zip(outs, (w, w2)):
                ref = o.nvfp4_quantize_for_gemm(full, True, True)
                keys = ["row_fp4", "row_sc"] + (["col_fp4", "col_sc"] if want_col else [])
                ok = ok and all(np.array_equal(got[i].numpy().reshape(ref[k].shape), ref[k]) for i, k in enumerate(keys))
                ok = ok and got[4].item() == ref["sg"] and (want_col or got[2] is None)
        outs = fsdp.all_gather_mxfp4_weights([shard, shard2], None, True, 1, quantize_shard=_oracle_mxfp4)
        for got, full in zip(outs, (w, w2)):
            ref = o.mxfp4_quantize_row_and_col(full, 1)
            ok = ok and all(np.array_equal(got[i].numpy().reshape(ref[k].shape), ref[k])
                            for i, k in enumerate(["row_fp4", "row_sc", "col_fp4", "col_sc"]))
        bad = False
        try:
            fsdp.all_gather_nvfp4_weight(shard[:100].contiguous(), None)
        except RuntimeError:
            bad = True
        q.put((rank, bool(ok), bad))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_packed_weight_all_gather_matches_full_quantisation():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=150) for _ in range(world)]
    for p in procs:
        p.join(30)
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] for r in res), "gathered operands differ from quantising the full weight"
    assert all(r[2] for r in res), "a shard with a row count that is not a multiple of 128 must be rejected"


def test_gathered_bytes_accounting():
    fsdp = importlib.import_module("mfu-fp4-training_b200.fsdp_weights")
    assert fsdp.gathered_bytes(4096, 4096, "nvfp4", False) == 4096 * 4096 * 9 // 16 + 4
    assert fsdp.gathered_bytes(4096, 4096, "mxfp4", True) == 2 * (4096 * 4096 // 2 + 4096 * 4096 // 32)
