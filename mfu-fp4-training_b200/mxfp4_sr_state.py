"""Checkpointable Philox coordinates for the stochastic-rounding MXFP4 producers.

Host-side mirror of the contract of the reference's ``low_bits_training/quantization/mxfp4_sr_state.py``
(class ``MXFP4SRState`` at :197-454, module helpers at :38-64 and :456-476): every stochastic producer of the
backward pass has a stable string key; a key owns one stream per rank, identified by

    seed        = (seed_base + rank * n_keys + slot + 1) mod 2^64      (slot = index of the key in sorted order)
    subsequence = subsequence_base + 2^32 * (number of reservations so far)

``reserve(key)`` hands out the next (seed, subsequence) pair, which is what ``mxfp4_quantize_for_gemm_opt`` and the
other ``*_opt`` quantisers of this package take as ``rng_seed`` / ``rng_subsequence``.  ``state_dict()`` gathers the
next subsequence of every key from every rank into one int64 tensor ``[world, n_keys, 2]`` with the same field names
as the reference's checkpoints, and ``load_state_dict`` refuses anything that would remap a stream (other world
size, other keys, seeds that do not follow from the base, subsequences off the stride).

The state lives in one int64 array; the seeds are derived, never stored.  Nothing here touches a GPU.
"""
from __future__ import annotations

import threading
from typing import Iterable, Mapping

import numpy as np
import torch
import torch.distributed as dist

CHECKPOINT_KEY = "mxfp4_sr_state"
STATE_VERSION = 1
SEED_NAMESPACE_VERSION = 1
SUBSEQUENCE_STRIDE = 1 << 32
UINT64_MAX = (1 << 64) - 1
DEFAULT_RESERVATION_MARGIN = 4096
MAX_RESERVATIONS_PER_PRODUCER_MICROBATCH = 3

_FIELDS = ("version", "seed_namespace_version", "seed_base", "subsequence_base", "subsequence_stride", "world_size",
           "rank_ids", "logical_keys", "states")


def _key(debug_name, role):
    if not isinstance(debug_name, str) or not debug_name:
        raise RuntimeError("checkpointed MXFP4 SR requires a non-empty stable _lbt_debug_name")
    return f"{debug_name}:sr:{role}"


def qkv_grad_key(debug_name):
    return _key(debug_name, "qkv_grad")


def wo_grad_key(debug_name):
    return _key(debug_name, "wo_grad")


def ffn_w2_grad_key(debug_name):
    return _key(debug_name, "ffn_w2_grad")


def ffn_deriv_grad_key(debug_name):
    return _key(debug_name, "ffn_deriv_grad")


def linear_grad_key(debug_name):
    return _key(debug_name, "linear_grad")


def _signed(v):
    v &= UINT64_MAX
    return v - (1 << 64) if v >> 63 else v


def _i64(values):
    return torch.tensor(list(values), dtype=torch.int64)


def _scalar(name, value):
    if not torch.is_tensor(value) or value.dtype != torch.int64 or value.numel() != 1:
        raise RuntimeError(f"MXFP4 SR checkpoint field {name!r} must be an int64 tensor with one value")
    return int(value.reshape(-1)[0].item())


class MXFP4SRState:
    """Rank-separated, per-producer advancing (seed, subsequence) pairs."""

    def __init__(self, logical_keys: Iterable[str], *, device="cpu", user_seed: int, user_subsequence_base: int,
                 training_steps: int, gradient_accumulation_steps: int,
                 reservation_margin: int = DEFAULT_RESERVATION_MARGIN, rank: int | None = None,
                 world_size: int | None = None) -> None:
        keys = tuple(sorted(set(logical_keys)))
        if not keys:
            raise ValueError("checkpointed MXFP4 SR requires at least one logical producer")
        for k in keys:
            if not isinstance(k, str) or not k:
                raise RuntimeError("checkpointed MXFP4 SR requires a non-empty stable _lbt_debug_name")
        self.logical_keys = keys
        self.device = torch.device(device)
        live = dist.is_available() and dist.is_initialized()
        here = (dist.get_rank(), dist.get_world_size()) if live else (0, 1)
        self.rank = here[0] if rank is None else int(rank)
        self.world_size = here[1] if world_size is None else int(world_size)
        if self.world_size <= 0 or not 0 <= self.rank < self.world_size:
            raise ValueError(f"MXFP4 SR rank must be in [0, world_size), got rank={self.rank}, world_size={self.world_size}")
        if live and (self.rank, self.world_size) != here:
            raise RuntimeError(f"MXFP4 SR rank/world namespace disagrees with the active process group: "
                               f"requested=({self.rank},{self.world_size}), actual={here}")
        self._check_same_keys_everywhere()
        for name, v in (("MXFP4_SR_SEED", user_seed), ("MXFP4_SR_SUBSEQUENCE", user_subsequence_base)):
            if not 0 <= int(v) <= UINT64_MAX:
                raise ValueError(f"{name} must be in [0, 2**64 - 1], got {v}")
        self.user_seed = int(user_seed)
        self._seed_base = self.user_seed
        self.user_subsequence_base = int(user_subsequence_base)
        steps, accum, margin = int(training_steps), int(gradient_accumulation_steps), int(reservation_margin)
        if steps < 0 or accum <= 0 or margin < 0:
            raise ValueError("invalid MXFP4 SR reservation horizon")
        self.reservations_per_slot = (steps + 1) * accum * MAX_RESERVATIONS_PER_PRODUCER_MICROBATCH + margin
        if self.user_subsequence_base > UINT64_MAX - self.reservations_per_slot * SUBSEQUENCE_STRIDE:
            raise ValueError(f"MXFP4_SR_SUBSEQUENCE leaves insufficient uint64 headroom: base={self.user_subsequence_base}, "
                             f"reservations={self.reservations_per_slot}")
        self._slot = {k: i for i, k in enumerate(keys)}
        self._taken = np.zeros(len(keys), dtype=np.int64)   # reservations made so far, per slot
        self._lock = threading.Lock()

    # ---- the streams ----------------------------------------------------------------------------------------
    def _seed_for(self, seed_base, rank, slot):
        return (int(seed_base) + rank * len(self.logical_keys) + slot + 1) & UINT64_MAX

    def _slot_of(self, key):
        try:
            return self._slot[key]
        except KeyError as exc:
            raise RuntimeError(f"unregistered MXFP4 SR logical identity {key!r}; the converted model/checkpoint "
                               "manifest is inconsistent") from exc

    def _next(self, slot):
        return self.user_subsequence_base + int(self._taken[slot]) * SUBSEQUENCE_STRIDE

    def reserve(self, logical_key: str) -> tuple[int, int]:
        """The next (seed, subsequence) of one producer; the one after it is 2^32 further on."""
        slot = self._slot_of(logical_key)
        with self._lock:
            sub = self._next(slot)
            if sub + SUBSEQUENCE_STRIDE > UINT64_MAX:
                raise OverflowError(f"MXFP4 SR subsequence exhausted for producer {logical_key!r}")
            self._taken[slot] += 1
        return self._seed_for(self._seed_base, self.rank, slot), sub

    def peek(self, logical_key: str) -> tuple[int, int]:
        slot = self._slot_of(logical_key)
        with self._lock:
            return self._seed_for(self._seed_base, self.rank, slot), self._next(slot)

    def reset_to_configured_base(self) -> None:
        self._seed_base = self.user_seed
        with self._lock:
            self._taken[:] = 0

    # ---- checkpoints ----------------------------------------------------------------------------------------
    def _check_same_keys_everywhere(self):
        if self.world_size == 1 or not (dist.is_available() and dist.is_initialized()):
            return
        seen = [None] * self.world_size
        dist.all_gather_object(seen, self.logical_keys)
        bad = [r for r, m in enumerate(seen) if not isinstance(m, (tuple, list)) or tuple(m) != self.logical_keys]
        if bad:
            raise RuntimeError(f"MXFP4 SR logical-producer manifests differ across ranks; local_rank={self.rank}, "
                               f"mismatched_ranks={bad}")

    def _local_rows(self):
        with self._lock:
            rows = [[_signed(self._seed_for(self._seed_base, self.rank, s)), _signed(self._next(s))]
                    for s in range(len(self.logical_keys))]
        return torch.tensor(rows, dtype=torch.int64, device=self.device)

    def _all_rows(self):
        local = self._local_rows()
        if self.world_size == 1:
            return local.unsqueeze(0).cpu()
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("multi-rank MXFP4 SR checkpoints require an initialized distributed process group")
        if (dist.get_rank(), dist.get_world_size()) != (self.rank, self.world_size):
            raise RuntimeError("MXFP4 SR rank/world changed after initialization")
        parts = [torch.empty_like(local) for _ in range(self.world_size)]
        dist.all_gather(parts, local)
        return torch.stack(parts).cpu()

    def state_dict(self) -> dict[str, object]:
        """Collective over the ranks when world_size > 1: every rank returns the whole table."""
        states = self._all_rows()
        return {"version": _i64([STATE_VERSION]), "seed_namespace_version": _i64([SEED_NAMESPACE_VERSION]),
                "seed_base": _i64([_signed(self._seed_base)]), "subsequence_base": _i64([_signed(self.user_subsequence_base)]),
                "subsequence_stride": _i64([SUBSEQUENCE_STRIDE]), "world_size": _i64([self.world_size]),
                "rank_ids": torch.arange(self.world_size, dtype=torch.int64), "logical_keys": list(self.logical_keys),
                "states": states.to(torch.int64).clone()}

    def load_state_dict(self, state_dict: Mapping[str, object]) -> None:
        if set(state_dict) != set(_FIELDS):
            raise RuntimeError(f"invalid MXFP4 SR checkpoint fields: expected={sorted(_FIELDS)}, got={sorted(state_dict)}")
        if (_scalar("version", state_dict["version"]) != STATE_VERSION
                or _scalar("seed_namespace_version", state_dict["seed_namespace_version"]) != SEED_NAMESPACE_VERSION):
            raise RuntimeError("unsupported MXFP4 SR checkpoint ABI")
        if _scalar("subsequence_stride", state_dict["subsequence_stride"]) != SUBSEQUENCE_STRIDE:
            raise RuntimeError("MXFP4 SR checkpoint stride differs from runtime")
        if _scalar("world_size", state_dict["world_size"]) != self.world_size:
            raise RuntimeError("MXFP4 SR checkpoint world_size differs from the runtime; refusing stream remap")
        ranks = state_dict["rank_ids"]
        if (not torch.is_tensor(ranks) or ranks.dtype != torch.int64
                or not torch.equal(ranks.cpu(), torch.arange(self.world_size, dtype=torch.int64))):
            raise RuntimeError("MXFP4 SR checkpoint rank namespace is malformed")
        if tuple(state_dict["logical_keys"]) != self.logical_keys:
            raise RuntimeError("MXFP4 SR logical-producer manifest differs from the checkpoint; refusing stream remap")
        states = state_dict["states"]
        shape = (self.world_size, len(self.logical_keys), 2)
        if not torch.is_tensor(states) or states.dtype != torch.int64 or tuple(states.shape) != shape:
            raise RuntimeError(f"invalid MXFP4 SR state matrix shape: expected {shape}")
        states = states.cpu()
        seed_base = _scalar("seed_base", state_dict["seed_base"]) & UINT64_MAX
        sub_base = _scalar("subsequence_base", state_dict["subsequence_base"]) & UINT64_MAX
        taken = np.zeros(len(self.logical_keys), dtype=np.int64)
        for r in range(self.world_size):
            for s in range(len(self.logical_keys)):
                if int(states[r, s, 0]) != _signed(self._seed_for(seed_base, r, s)):
                    raise RuntimeError("MXFP4 SR checkpoint seed namespace is inconsistent; refusing resume")
                nxt = int(states[r, s, 1]) & UINT64_MAX
                if nxt < sub_base:
                    raise RuntimeError("MXFP4 SR checkpoint subsequence precedes its base")
                if (nxt - sub_base) % SUBSEQUENCE_STRIDE:
                    raise RuntimeError("MXFP4 SR checkpoint subsequence is not stride-aligned")
                if r == self.rank:
                    taken[s] = (nxt - sub_base) // SUBSEQUENCE_STRIDE
        self._seed_base, self.user_subsequence_base = seed_base, sub_base
        with self._lock:
            self._taken[:] = taken


_ACTIVE: MXFP4SRState | None = None


def active_mxfp4_sr_state() -> MXFP4SRState | None:
    return _ACTIVE


def set_active_mxfp4_sr_state(state: MXFP4SRState | None) -> None:
    global _ACTIVE
    _ACTIVE = state


def reserve_mxfp4_sr(logical_key: str | None) -> tuple[int, int]:
    """reserve() on the installed state (reference :465-476); raises when there is no key or no state."""
    if not logical_key:
        raise RuntimeError("ranked row-gradient MXFP4 SR reached a quantizer without a stable producer key")
    if _ACTIVE is None:
        raise RuntimeError("ranked row-gradient MXFP4 SR has no active checkpointed state; install it through the "
                           "trainer before the first backward")
    return _ACTIVE.reserve(logical_key)
