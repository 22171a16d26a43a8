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

``all_gather_nvfp4_weights`` / ``all_gather_mxfp4_weights`` do the same for a LIST of weights (a layer's) with one
``all_reduce(MAX)`` over the stacked amaxes and one coalesced group of all-gathers: the exchange is bound by the
number of small collectives, not by NVLink bandwidth (99 MB per rank for the three FFN weights).

Gathered buffers live in local HBM before any GEMM touches them; no kernel reads peer memory.
Shards must have a multiple of 128 rows.  ``quantize_shard`` is injectable so that the exchange
logic can be exercised on CPU ranks (gloo) with a stand-in quantiser.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def _part_shapes(N: int, K: int, fmt: str, want_col: bool):
    """Shapes of (row_fp4, row_sc, col_fp4, col_sc) of a [N, K] shard."""
    kb = 64 if fmt == "nvfp4" else 128
    shapes = [(N, K // 2), (N // 128, K // kb, 512)]
    if want_col:
        shapes += [(K, N // 2), (K // 128, N // kb, 512)]
    return shapes


def _cuda_quantize_nvfp4(w_shard: torch.Tensor, amax: torch.Tensor, encode_centric: bool, want_col: bool, out=None,
                         weight_2d: bool = False):
    """Row (+column) NVFP4 quantisation of a shard with a given device-resident tensor amax; into `out`
    (row_fp4, row_sc[, col_fp4, col_sc]) when given.  ``weight_2d``: one decode-centric scale per 16 x 16 tile for both
    orientations (tk_quantize_weight_2d's blocks; needs both orientations)."""
    from . import _lib
    N, K = w_shard.shape
    u8 = dict(dtype=torch.uint8, device=w_shard.device)
    if out is None:
        out = [torch.empty(sh, **u8) for sh in _part_shapes(N, K, "nvfp4", want_col)]
    row_fp4, row_sc = out[0], out[1]
    col_fp4, col_sc = (out[2], out[3]) if want_col else (None, None)
    if weight_2d:
        if not want_col:
            raise RuntimeError("2-D weight blocks are quantised in both orientations at once")
        with torch.cuda.device(w_shard.device):
            _lib.call("fp4b200_nvfp4_quantize_weight_2d_with_amax", w_shard.data_ptr(), N, K, amax.data_ptr(),
                      row_fp4.data_ptr(), row_sc.data_ptr(), col_fp4.data_ptr(), col_sc.data_ptr(),
                      torch.cuda.current_stream(w_shard.device).cuda_stream)
        return row_fp4, row_sc, col_fp4, col_sc
    with torch.cuda.device(w_shard.device):
        _lib.call("fp4b200_nvfp4_quantize", w_shard.data_ptr(), N, K, amax.data_ptr(), None, int(encode_centric),
                  row_fp4.data_ptr(), row_sc.data_ptr(), None if col_fp4 is None else col_fp4.data_ptr(),
                  None if col_sc is None else col_sc.data_ptr(), None,
                  torch.cuda.current_stream(w_shard.device).cuda_stream)
    return row_fp4, row_sc, col_fp4, col_sc


def _cuda_quantize_mxfp4(w_shard: torch.Tensor, mode: int, want_col: bool, out=None):
    from . import _lib
    N, K = w_shard.shape
    u8 = dict(dtype=torch.uint8, device=w_shard.device)
    if out is None:
        out = [torch.empty(sh, **u8) for sh in _part_shapes(N, K, "mxfp4", want_col)]
    row_fp4, row_sc = out[0], out[1]
    col_fp4, col_sc = (out[2], out[3]) if want_col else (None, None)
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


def _local_amaxes(shards):
    """Tensor maxima of the shards as one float32 vector on their device: the library's amax kernel on CUDA, torch
    on CPU (the gloo tests)."""
    if shards[0].is_cuda:
        from . import _lib
        buf = torch.empty((len(shards), 2), dtype=torch.float32, device=shards[0].device)
        with torch.cuda.device(shards[0].device):
            st = torch.cuda.current_stream(shards[0].device).cuda_stream
            for i, w in enumerate(shards):
                _lib.call("fp4b200_nvfp4_amax", w.data_ptr(), w.numel(), buf[i].data_ptr(), st)
        return buf[:, 0].contiguous()
    return torch.stack([w.abs().amax().to(torch.float32) for w in shards])


# Send and receive buffers of the list gathers, kept per (format, shard shapes, orientation, device, world) when the
# caller asks for it: a layer's gather runs every step with the same shapes, and fresh 100 MB blocks that have been
# used on the collective's stream come back from the caching allocator slowly (milliseconds against 0.3 ms of work).
_WORKSPACES = {}


def _workspace(fmt, w_shards, want_col, world):
    key = (fmt, tuple(tuple(w.shape) for w in w_shards), bool(want_col), str(w_shards[0].device), world)
    ws = _WORKSPACES.get(key)
    if ws is None:
        u8 = dict(dtype=torch.uint8, device=w_shards[0].device)
        send = [[torch.empty(sh, **u8) for sh in _part_shapes(w.shape[0], w.shape[1], fmt, want_col)] for w in w_shards]
        recv = [torch.empty((world,) + tuple(t.shape), **u8) for parts in send for t in parts]
        ws = _WORKSPACES[key] = (send, recv)
    return ws


def _gather_parts(parts, group, world, outs=None):
    """All-gathers every tensor of `parts` (rank-major, a new leading dimension of `world`), as ONE group of
    collectives where the backend can coalesce them (NCCL), else one call each."""
    if outs is None:
        outs = [torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device) for t in parts]
    coalesce = parts[0].is_cuda and hasattr(dist, "_coalescing_manager")
    if coalesce:
        with dist._coalescing_manager(group=group, device=parts[0].device, async_ops=False):
            for o, t in zip(outs, parts):
                dist.all_gather_into_tensor(o, t.contiguous().unsqueeze(0), group=group)
    else:
        for o, t in zip(outs, parts):
            dist.all_gather_into_tensor(o, t.contiguous().unsqueeze(0), group=group)
    return outs


def _assemble(gathered, want_col):
    """(row_fp4, row_sc, col_fp4, col_sc) of the full weight from the rank-major gathers of a shard's four parts: the
    row-wise parts concatenate along their leading dimension (a view), the column-wise ones along their second (one
    permuting copy each)."""
    row_fp4, row_sc = (g.reshape((g.shape[0] * g.shape[1],) + tuple(g.shape[2:])) for g in gathered[:2])
    col_fp4 = col_sc = None
    if want_col:
        col_fp4, col_sc = (g.movedim(0, 1).reshape((g.shape[1], g.shape[0] * g.shape[2]) + tuple(g.shape[3:])).contiguous()
                           for g in gathered[2:4])
    return row_fp4, row_sc, col_fp4, col_sc


def all_gather_nvfp4_weights(w_shards, group=None, want_col: bool = True, encode_centric: bool = True,
                             quantize_shard: Optional[Callable] = None, reuse_buffers: bool = False,
                             weight_2d: bool = False):
    """``all_gather_nvfp4_weight`` for a list of weights with one amax all-reduce and one group of all-gathers.
    Returns a list of ``(row_fp4, row_sc, col_fp4, col_sc, sg [1])``, byte-identical to the per-weight function's.
    ``reuse_buffers``: the results live in a workspace kept for these shapes and are overwritten by the next call
    with the same shapes (what a layer's per-step gather wants); off, every call returns fresh tensors.
    ``weight_2d``: the weights' 16 x 16 block form (tk_quantize_weight_2d, fused_te_linear.py:4716-4748: decode-centric,
    one scale per tile for both orientations); shards of a multiple of 128 rows hold whole tiles, so the gathered
    bytes are those of quantising the gathered weight."""
    if weight_2d and quantize_shard is None:
        def quantize_shard_2d(w, amax, ec, wc, out=None):
            return _cuda_quantize_nvfp4(w, amax, ec, wc, out=out, weight_2d=True)
    else:
        quantize_shard_2d = None
    for w in w_shards:
        _check_shard(w)
    world = dist.get_world_size(group)
    amaxes = _local_amaxes(w_shards)
    dist.all_reduce(amaxes, op=dist.ReduceOp.MAX, group=group)
    q = quantize_shard or quantize_shard_2d or _cuda_quantize_nvfp4
    n_parts = 4 if want_col else 2
    send, recv = (_workspace("nvfp4", w_shards, want_col, world) if (reuse_buffers and quantize_shard is None)
                  else ([None] * len(w_shards), None))
    parts = []
    for i, w in enumerate(w_shards):
        got = q(w, amaxes[i:i + 1], encode_centric, want_col) if send[i] is None else \
            q(w, amaxes[i:i + 1], encode_centric, want_col, out=send[i])
        parts.extend(got[:n_parts])
    gathered = _gather_parts(parts, group, world, recv)
    out = []
    for i in range(len(w_shards)):
        out.append(_assemble(gathered[i * n_parts:(i + 1) * n_parts], want_col) + (amaxes[i:i + 1] / 2688.0,))
    return out


def all_gather_mxfp4_weights(w_shards, group=None, want_col: bool = True, mode: int = 1,
                             quantize_shard: Optional[Callable] = None, reuse_buffers: bool = False):
    """``all_gather_mxfp4_weight`` for a list of weights with one group of all-gathers; returns a list of
    ``(row_fp4, row_sc, col_fp4, col_sc)``.  ``reuse_buffers`` as in ``all_gather_nvfp4_weights`` (the column-wise
    results are permuted copies and always fresh)."""
    for w in w_shards:
        _check_shard(w)
    world = dist.get_world_size(group)
    q = quantize_shard or _cuda_quantize_mxfp4
    n_parts = 4 if want_col else 2
    send, recv = (_workspace("mxfp4", w_shards, want_col, world) if (reuse_buffers and quantize_shard is None)
                  else ([None] * len(w_shards), None))
    parts = []
    for i, w in enumerate(w_shards):
        got = q(w, mode, want_col) if send[i] is None else q(w, mode, want_col, out=send[i])
        parts.extend(got[:n_parts])
    gathered = _gather_parts(parts, group, world, recv)
    return [_assemble(gathered[i * n_parts:(i + 1) * n_parts], want_col) for i in range(len(w_shards))]
