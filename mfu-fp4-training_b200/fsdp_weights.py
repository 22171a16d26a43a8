"""All-gather of FSDP-sharded weights as packed FP4 + scales instead of BF16.

The token dimension M is what the hot path shards across GPUs (no collective inside fprop/dgrad);
the one exchange step is bringing every rank's weight shard to every rank.  The reference gathers
BF16 parameters and re-quantises the full weight on every rank each step; its only packed
precedent is TE's ``NVFP4Tensor.fsdp_pre_all_gather/post_all_gather``
(TransformerEngine/transformer_engine/pytorch/tensor/nvfp4_tensor.py:555-660).  Here each rank
quantises only its own ``[N/G, K]`` shard and the ranks exchange 0.5625 B (NVFP4) or 0.53 B (MXFP4)
per parameter and orientation instead of 2 B:

1. NVFP4 only: local tensor amax, ``all_reduce(MAX)`` of one float, so that every shard is
   quantised with the amax of the whole weight (required for byte equality with quantising the
   gathered BF16 weight);
2. quantise the shard row-wise and column-wise with that amax;
3. ``all_gather_into_tensor`` of codes and scale tiles.  Row-wise payloads are sharded along their
   leading dimension and the scale tiles are tile-major, so shards concatenate byte-contiguously.
   Column-wise payloads ``[K, N/2]`` / ``[K/128, N/64, 512]`` are sharded along their second
   dimension: they are gathered rank-major and permuted once on the device.

Gathered buffers live in local HBM before any GEMM touches them; no kernel reads peer memory.
Shards must have a multiple of 128 rows.  ``quantize_shard`` is injectable so that the exchange
logic can be exercised on CPU ranks (gloo) with a stand-in quantiser.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def _cuda_quantize_nvfp4(w_shard: torch.Tensor, amax: torch.Tensor, encode_centric: bool, want_col: bool):
    """Row (+column) NVFP4 quantisation of a shard with a given device-resident tensor amax."""
    from . import _lib
    N, K = w_shard.shape
    u8 = dict(dtype=torch.uint8, device=w_shard.device)
    row_fp4 = torch.empty((N, K // 2), **u8)
    row_sc = torch.empty((N // 128, K // 64, 512), **u8)
    col_fp4 = torch.empty((K, N // 2), **u8) if want_col else None
    col_sc = torch.empty((K // 128, N // 64, 512), **u8) if want_col else None
    with torch.cuda.device(w_shard.device):
        _lib.call("fp4b200_nvfp4_quantize", w_shard.data_ptr(), N, K, amax.data_ptr(), None, int(encode_centric),
                  row_fp4.data_ptr(), row_sc.data_ptr(), None if col_fp4 is None else col_fp4.data_ptr(),
                  None if col_sc is None else col_sc.data_ptr(), None,
                  torch.cuda.current_stream(w_shard.device).cuda_stream)
    return row_fp4, row_sc, col_fp4, col_sc


def _cuda_quantize_mxfp4(w_shard: torch.Tensor, mode: int, want_col: bool):
    from . import _lib
    N, K = w_shard.shape
    u8 = dict(dtype=torch.uint8, device=w_shard.device)
    row_fp4 = torch.empty((N, K // 2), **u8)
    row_sc = torch.empty((N // 128, K // 128, 512), **u8)
    col_fp4 = torch.empty((K, N // 2), **u8) if want_col else None
    col_sc = torch.empty((K // 128, N // 128, 512), **u8) if want_col else None
    with torch.cuda.device(w_shard.device):
        _lib.call("fp4b200_mxfp4_quantize", w_shard.data_ptr(), N, K, int(mode), row_fp4.data_ptr(),
                  row_sc.data_ptr(), None if col_fp4 is None else col_fp4.data_ptr(),
                  None if col_sc is None else col_sc.data_ptr(),
                  torch.cuda.current_stream(w_shard.device).cuda_stream)
    return row_fp4, row_sc, col_fp4, col_sc


def _gather_dim0(t: torch.Tensor, group, world: int) -> torch.Tensor:
    out = torch.empty((world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out


def _gather_dim1(t: torch.Tensor, group, world: int) -> torch.Tensor:
    """Gathers shards that split the SECOND dimension: rank-major gather, then one permute-copy."""
    g = _gather_dim0(t.unsqueeze(0), group, world)            # [G, d0, d1/G, ...]
    g = g.movedim(0, 1)                                        # [d0, G, d1/G, ...]
    return g.reshape((t.shape[0], world * t.shape[1]) + tuple(t.shape[2:])).contiguous()


def _check_shard(w_shard: torch.Tensor):
    if w_shard.dim() != 2 or w_shard.dtype != torch.bfloat16 or not w_shard.is_contiguous():
        raise RuntimeError("weight shard must be a contiguous 2-D bfloat16 tensor [N/G, K]")
    if w_shard.shape[0] % 128 or w_shard.shape[1] % 128:
        raise RuntimeError(f"weight shard {tuple(w_shard.shape)}: rows and K must be multiples of 128")


def gathered_bytes(N: int, K: int, fmt: str = "nvfp4", want_col: bool = True) -> int:
    """Bytes every rank receives for one weight ``[N, K]`` (both orientations when ``want_col``)."""
    per = N * K // 2 + N * K // (16 if fmt == "nvfp4" else 32)
    return per * (2 if want_col else 1) + (4 if fmt == "nvfp4" else 0)


def all_gather_nvfp4_weight(w_shard: torch.Tensor, group=None, want_col: bool = True, encode_centric: bool = True,
                            quantize_shard: Optional[Callable] = None):
    """Returns ``(row_fp4 [N,K/2], row_sc [N/128,K/64,512], col_fp4 [K,N/2], col_sc [K/128,N/64,512], sg [1])``
    for the full weight, byte-identical on every rank to quantising the gathered BF16 weight."""
    _check_shard(w_shard)
    world = dist.get_world_size(group)
    amax = w_shard.abs().amax().to(torch.float32).reshape(1)
    dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    q = quantize_shard or _cuda_quantize_nvfp4
    row_fp4, row_sc, col_fp4, col_sc = q(w_shard, amax, encode_centric, want_col)
    row_fp4 = _gather_dim0(row_fp4, group, world)
    row_sc = _gather_dim0(row_sc, group, world)
    if want_col:
        col_fp4 = _gather_dim1(col_fp4, group, world)
        col_sc = _gather_dim1(col_sc, group, world)
    sg = amax / 2688.0
    return row_fp4, row_sc, col_fp4, col_sc, sg


def all_gather_mxfp4_weight(w_shard: torch.Tensor, group=None, want_col: bool = True, mode: int = 1,
                            quantize_shard: Optional[Callable] = None):
    """MXFP4 counterpart (no tensor-level scale, hence no amax exchange): returns
    ``(row_fp4, row_sc [N/128,K/128,512], col_fp4, col_sc [K/128,N/128,512])``."""
    _check_shard(w_shard)
    world = dist.get_world_size(group)
    q = quantize_shard or _cuda_quantize_mxfp4
    row_fp4, row_sc, col_fp4, col_sc = q(w_shard, mode, want_col)
    row_fp4 = _gather_dim0(row_fp4, group, world)
    row_sc = _gather_dim0(row_sc, group, world)
    if want_col:
        col_fp4 = _gather_dim1(col_fp4, group, world)
        col_sc = _gather_dim1(col_sc, group, world)
    return row_fp4, row_sc, col_fp4, col_sc
