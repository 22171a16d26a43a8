"""GPU, two ranks over NCCL (skipped on a single-GPU box): the packed-weight all-gather through the
CUDA quantiser equals quantising the full weight locally, byte for byte, on every rank."""
import importlib
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        fsdp = importlib.import_module("mfu-fp4-training_b200.fsdp_weights")
        tkq = importlib.import_module("mfu-fp4-training_b200.tk_quant_v5")
        mxq = importlib.import_module("mfu-fp4-training_b200.mxfp4_quant_v4")
        N, K = 1024, 512
        g = torch.Generator().manual_seed(3)
        w = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
        w[700, 3] = 0.75
        wd = w.cuda()
        shard = wd[rank * N // world:(rank + 1) * N // world].contiguous()
        out = fsdp.all_gather_nvfp4_weight(shard, None, True, True)
        ref = tkq.tk_quantize_for_gemm(wd, True, True)
        ok = all(torch.equal(out[i].reshape(-1), ref[i].view(torch.uint8).reshape(-1)) for i in range(4))
        ok = ok and out[4].item() == ref[4].item()
        out = fsdp.all_gather_mxfp4_weight(shard, None, True, 1)
        ref = mxq.mxfp4_quantize_row_and_col(wd, 1)
        ok = ok and all(torch.equal(out[i].reshape(-1), ref[i].view(torch.uint8).reshape(-1)) for i in range(4))
        # a layer's weights at once (one amax all-reduce, one group of all-gathers)
        w2 = (0.03 * torch.randn(512, 768, generator=g)).to(torch.bfloat16)
        w2[9, 9] = -0.9
        w2d = w2.cuda()
        shard2 = w2d[rank * 512 // world:(rank + 1) * 512 // world].contiguous()
        for want_col in (True, False):
            outs = fsdp.all_gather_nvfp4_weights([shard, shard2], None, want_col, True)
            for got, full in zip(outs, (wd, w2d)):
                ref = tkq.tk_quantize_for_gemm(full, True, True)
                ok = ok and all(torch.equal(got[i].reshape(-1), ref[i].view(torch.uint8).reshape(-1)) for i in range(4 if want_col else 2))
                ok = ok and got[4].item() == ref[4].item()
        for _ in range(2):   # the kept send / receive buffers give the same bytes on every call
            outs = fsdp.all_gather_nvfp4_weights([shard, shard2], None, True, True, reuse_buffers=True)
            for got, full in zip(outs, (wd, w2d)):
                ref = tkq.tk_quantize_for_gemm(full, True, True)
                ok = ok and all(torch.equal(got[i].reshape(-1), ref[i].view(torch.uint8).reshape(-1)) for i in range(4))
        # the weights' 16 x 16 block form: shards hold whole tiles, so the gather equals tk_quantize_weight_2d of the weight
        outs = fsdp.all_gather_nvfp4_weights([shard, shard2], None, True, False, weight_2d=True)
        for got, full in zip(outs, (wd, w2d)):
            ref = tkq.tk_quantize_weight_2d(full)
            ok = ok and all(torch.equal(got[i].reshape(-1), ref[i].view(torch.uint8).reshape(-1)) for i in range(4))
            ok = ok and got[4].item() == ref[4].item()
        outs = fsdp.all_gather_mxfp4_weights([shard, shard2], None, True, 1)
        for got, full in zip(outs, (wd, w2d)):
            ref = mxq.mxfp4_quantize_row_and_col(full, 1)
            ok = ok and all(torch.equal(got[i].reshape(-1), ref[i].view(torch.uint8).reshape(-1)) for i in range(4))
        torch.cuda.synchronize()
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_packed_weight_all_gather_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(2)]
    for p in procs:
        p.join(30)
    assert all(r[1] for r in res)
