"""Checkpointable, device-resident Philox coordinates: one (seed, next subsequence) pair per backward producer.

Host-side mirror of the contract of the reference's ``low_bits_training/quantization/localcta_sr_state.py``
(class ``LocalCTASRState`` at :250-606, key helpers :36-57, enable policy :60-116, trainer / checkpointer hooks
:609-902).  Every stochastic producer of the backward pass has a stable string key; the key owns one persistent
``int64[2]`` on the producer's device,

    [0] seed            = (seed_base + rank * n_keys + slot + 1) mod 2^64   (slot = index of the key in sorted order)
    [1] next subsequence, starting at the configured base; the CONSUMER adds 2^32 per reserved launch, on its own
        CUDA stream, right before the quantiser it feeds

so that the numbering depends neither on the Python launch order of different producers nor on how their streams
overlap, and a captured CUDA graph keeps advancing it on every replay.  Here all pairs are the rows of ONE int64
tensor ``[n_keys, 2]`` (``get(key)`` is a view of a row): one allocation, one copy per checkpoint.  The consumer in
this package is ``fp4b200_sr_reserve_from_state`` (``tk_quant_v5.producer_sr_state``), which hands the pair to the
stochastic quantiser launched next and advances the row.

``state_dict()`` gathers every rank's rows into ``[world, n_keys, 2]`` under the reference's field names (version 2);
``load_state_dict`` refuses whatever would remap a stream (other world size, other keys, seeds that do not follow
from the base); ``migrate_from_v1_state_dict`` takes the older one-table format ``[n_keys, 2]`` on request.
"""
from __future__ import annotations

import os
import types
from contextlib import contextmanager
from typing import Iterable, Iterator, Mapping

import torch
import torch.distributed as dist

CHECKPOINT_KEY = "localcta_sr_state"
LEGACY_STATE_VERSION = 1
STATE_VERSION = 2
SEED_NAMESPACE_VERSION = 1
SUBSEQUENCE_STRIDE = 1 << 32
UINT64_MAX = (1 << 64) - 1
DEFAULT_RESERVATION_MARGIN = 4096
V1_MIGRATION_ENV = "LBT_LOCALCTA_SR_V1_MIGRATION"
V1_RANK_NAMESPACE_MIGRATION = "rank_namespace_v2"
V1_EXPECTED_WORLD_SIZE_ENV = "LBT_LOCALCTA_SR_V1_EXPECTED_WORLD_SIZE"

_V2_FIELDS = frozenset(("version", "seed_namespace_version", "seed_base", "subsequence_stride", "world_size",
                        "rank_ids", "logical_keys", "states"))
_V1_FIELDS = frozenset(("version", "subsequence_stride", "logical_keys", "states"))
_FFN_MODULES = frozenset(("FusedFeedForwardFP4_TK", "FusedSquaredReLUFeedForwardFP4_TK"))
_ATTENTION_MODULES = frozenset(("FusedAttentionFP4_TK",))


# ---- keys --------------------------------------------------------------------------------------------------------

def _named(debug_name):
    if not isinstance(debug_name, str) or not debug_name:
        raise RuntimeError("checkpointed localCTA SR requires a non-empty stable _lbt_debug_name")
    return debug_name


def ffn_w2_grad_key(debug_name: str) -> str:
    return f"{_named(debug_name)}:sr:ffn_w2_grad"


def ffn_deriv_grad_key(debug_name: str) -> str:
    return f"{_named(debug_name)}:sr:ffn_deriv_grad"


def qkv_grad_key(debug_name: str) -> str:
    return f"{_named(debug_name)}:sr:qkv_grad"


def wo_grad_key(debug_name: str) -> str:
    return f"{_named(debug_name)}:sr:wo_grad"


def discover_logical_keys(model_parts: Iterable[torch.nn.Module]) -> tuple[str, ...]:
    """The producers of a converted model (reference :216-247): every fused FFN module owns a W2-gradient and an
    activation-derivative-gradient producer, every fused attention module a QKV-gradient and an output-projection
    one; modules are told apart by their ``_lbt_debug_name``, and two modules under one name are refused."""
    owner: dict[str, int] = {}
    for part in model_parts:
        for module in part.modules():
            kind = type(module).__name__
            if kind in _FFN_MODULES:
                base = _named(getattr(module, "_lbt_debug_name", None))
                keys = (ffn_w2_grad_key(base), ffn_deriv_grad_key(base))
            elif kind in _ATTENTION_MODULES:
                base = _named(getattr(module, "_lbt_debug_name", None))
                keys = (qkv_grad_key(f"{base}:qkv"), wo_grad_key(f"{base}:wo"))
            else:
                continue
            for key in keys:
                if owner.setdefault(key, id(module)) != id(module):
                    raise RuntimeError(f"duplicate localCTA SR logical identity {key!r}; converted modules must have "
                                       "unique stable _lbt_debug_name values")
    return tuple(sorted(owner))


# ---- enable policy (environment) ---------------------------------------------------------------------------------

def _flag(name, default=False):
    raw = os.environ.get(name)
    return default if raw is None else raw.strip().lower() not in ("", "0", "false", "no", "off")


def _localcta_v4_enabled() -> bool:
    return _flag("USE_TK_LOCALCTA") and os.environ.get("USE_TK_LOCALCTA_VARIANT", "v1").strip().lower() == "v4"


def _role_scale_sr_enabled(role: str) -> bool:
    """Scale SR of a role: its own switch if set; else the global scale switch, which an explicit data switch of the
    role narrows to that switch's value."""
    role = role.upper()
    if os.environ.get(f"NVFP4_SCALE_SR_{role}") is not None:
        return _flag(f"NVFP4_SCALE_SR_{role}")
    if not _flag("NVFP4_USE_SCALE_STOCHASTIC_ROUNDING"):
        return False
    return _flag(f"NVFP4_SR_{role}") if os.environ.get(f"NVFP4_SR_{role}") is not None else True


def _role_sr_enabled(role: str) -> bool:
    """Does the role draw random words at all (data SR or scale SR)?  Data SR: the role's switch, else the global
    one; for gradients additionally the axes setting must not be none."""
    role = role.upper()
    own = os.environ.get(f"NVFP4_SR_{role}")
    data = _flag(f"NVFP4_SR_{role}") if own is not None else _flag("NVFP4_USE_STOCHASTIC_ROUNDING")
    if role == "GRAD":
        axes = os.environ.get("NVFP4_GRAD_SR_AXES", "both").strip().lower().replace("-", "_")
        data = data and axes not in ("none", "off", "0")
    return data or _role_scale_sr_enabled(role)


def localcta_v4_grad_sr_enabled() -> bool:
    return _localcta_v4_enabled() and _role_sr_enabled("grad")


# ---- integer helpers ---------------------------------------------------------------------------------------------

def _signed(value: int) -> int:
    value &= UINT64_MAX
    return value - (1 << 64) if value >> 63 else value


def _i64(values) -> torch.Tensor:
    return torch.tensor(list(values), dtype=torch.int64)


def _field(name, value) -> torch.Tensor:
    if not torch.is_tensor(value) or value.dtype != torch.int64:
        raise RuntimeError(f"localCTA SR checkpoint field {name!r} must be an int64 tensor")
    return value.detach().cpu()


def _scalar(name, value) -> int:
    t = _field(name, value)
    if t.numel() != 1:
        raise RuntimeError(f"localCTA SR checkpoint field {name!r} must contain one value")
    return int(t.reshape(-1)[0].item())


def _u64_setting(name, value) -> int:
    value = int(value)
    if not 0 <= value <= UINT64_MAX:
        raise ValueError(f"{name} must be in [0, 2**64 - 1], got {value}")
    return value


def _reservation_horizon(base, training_steps, gradient_accumulation_steps, reservation_margin) -> int:
    """One reservation per producer and micro-batch, one optimizer step to spare, plus the margin (reference
    :152-184); the whole span must fit under 2^64 above the base."""
    steps, accum, margin = int(training_steps), int(gradient_accumulation_steps), int(reservation_margin)
    if steps < 0:
        raise ValueError(f"training_steps must be non-negative, got {steps}")
    if accum <= 0:
        raise ValueError(f"gradient_accumulation_steps must be positive, got {accum}")
    if margin < 0:
        raise ValueError(f"reservation_margin must be non-negative, got {margin}")
    reservations = (steps + 1) * accum + margin
    if base > UINT64_MAX - reservations * SUBSEQUENCE_STRIDE:
        raise ValueError(f"NVFP4_RNG_SUBSEQUENCE_BASE leaves insufficient uint64 headroom: base={base}, "
                         f"reservations={reservations}, stride={SUBSEQUENCE_STRIDE}, "
                         f"required_span={reservations * SUBSEQUENCE_STRIDE}")
    return reservations


def _rank_and_world(rank, world_size):
    live = dist.is_available() and dist.is_initialized()
    here = (dist.get_rank(), dist.get_world_size()) if live else (0, 1)
    r = here[0] if rank is None else int(rank)
    w = here[1] if world_size is None else int(world_size)
    if w <= 0:
        raise ValueError(f"localCTA SR world_size must be positive, got {w}")
    if not 0 <= r < w:
        raise ValueError(f"localCTA SR rank must be in [0, world_size), got rank={r}, world_size={w}")
    if live and (r, w) != here:
        raise RuntimeError(f"localCTA SR rank/world namespace disagrees with the active process group: "
                           f"requested=({r},{w}), actual=({here[0]},{here[1]})")
    return r, w


# ---- the table ---------------------------------------------------------------------------------------------------

class LocalCTASRState:
    """Per-rank table of (seed, next subsequence) rows, one per producer key, resident on the producers' device."""

    def __init__(self, logical_keys: Iterable[str], *, device, user_seed: int, user_subsequence_base: int,
                 training_steps: int, gradient_accumulation_steps: int,
                 reservation_margin: int = DEFAULT_RESERVATION_MARGIN, rank: int | None = None,
                 world_size: int | None = None) -> None:
        keys = tuple(sorted(set(logical_keys)))
        if not keys:
            raise ValueError("checkpointed localCTA SR requires at least one logical producer")
        for key in keys:
            _named(key)
        self.logical_keys = keys
        self.device = torch.device(device)
        self.rank, self.world_size = _rank_and_world(rank, world_size)
        self._check_same_keys_everywhere()
        self.user_seed = _u64_setting("NVFP4_RNG_SEED", user_seed)
        self._seed_base = self.user_seed
        self.user_subsequence_base = _u64_setting("NVFP4_RNG_SUBSEQUENCE_BASE", user_subsequence_base)
        self.reservations_per_slot = _reservation_horizon(self.user_subsequence_base, training_steps,
                                                          gradient_accumulation_steps, reservation_margin)
        self._slot = {key: i for i, key in enumerate(keys)}
        self._table = self._fresh_rows(self.user_seed, [self.user_subsequence_base] * len(keys)).to(self.device)

    # ---- rows ----
    def _seed_for(self, seed_base: int, rank: int, slot: int) -> int:
        return (int(seed_base) + rank * len(self.logical_keys) + slot + 1) & UINT64_MAX

    def _fresh_rows(self, seed_base, next_subsequences) -> torch.Tensor:
        return torch.tensor([[_signed(self._seed_for(seed_base, self.rank, s)), _signed(int(n))]
                             for s, n in enumerate(next_subsequences)], dtype=torch.int64)

    def _local_state_matrix(self) -> torch.Tensor:
        return self._table

    def get(self, logical_key: str, device=None) -> torch.Tensor:
        """The producer's persistent int64[2] (a row of the table; the consumer advances it in place)."""
        slot = self._slot.get(logical_key)
        if slot is None:
            raise RuntimeError(f"unregistered localCTA SR logical identity {logical_key!r}; the converted "
                               "model/checkpoint manifest is inconsistent")
        if device is not None and torch.device(device) != self._table.device:
            raise RuntimeError(f"localCTA SR state {logical_key!r} is on {self._table.device}, but its producer is on "
                               f"{torch.device(device)}")
        return self._table[slot]

    def _drain(self) -> None:
        # checkpoint / capture boundaries only: waits for every stream's pending advances (and graph replays)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _write_rows(self, rows: torch.Tensor) -> None:
        self._table.copy_(rows.to(self.device))
        self._drain()

    def reset_to_configured_base(self) -> None:
        """A deliberate new phase from the configured seed and base."""
        self._drain()
        self._seed_base = self.user_seed
        self._write_rows(self._fresh_rows(self.user_seed, [self.user_subsequence_base] * len(self.logical_keys)))

    @contextmanager
    def preserve_during_cuda_graph_capture(self, logical_keys: Iterable[str]) -> Iterator[None]:
        """Rolls back what warm-up and capture runs reserved for these keys; the captured kernels keep pointing at
        the live rows and advance them on every real replay."""
        slots = [self._slot_checked(key) for key in dict.fromkeys(logical_keys)]
        if not slots:
            yield
            return
        self._drain()
        kept = self._table[slots].clone()
        self._drain()
        try:
            yield
        finally:
            self._drain()
            self._table[slots] = kept
            self._drain()

    def _slot_checked(self, key):
        self.get(key)
        return self._slot[key]

    # ---- checkpoints ----
    def _check_same_keys_everywhere(self) -> None:
        if self.world_size == 1 or not (dist.is_available() and dist.is_initialized()):
            return
        seen: list[object] = [None] * self.world_size
        dist.all_gather_object(seen, self.logical_keys)
        bad = [r for r, m in enumerate(seen) if not isinstance(m, (tuple, list)) or tuple(m) != self.logical_keys]
        if bad:
            raise RuntimeError(f"localCTA SR logical-producer manifests differ across ranks; local_rank={self.rank}, "
                               f"mismatched_ranks={bad}")

    def _gather_rank_states(self) -> torch.Tensor:
        self._drain()
        local = self._table.detach().clone()
        if self.world_size == 1:
            return local.unsqueeze(0).cpu()
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("multi-rank localCTA SR checkpoints require an initialized distributed process group")
        here = (dist.get_rank(), dist.get_world_size())
        if here != (self.rank, self.world_size):
            raise RuntimeError(f"localCTA SR rank/world changed after initialization: state=({self.rank},"
                               f"{self.world_size}), process_group=({here[0]},{here[1]})")
        parts = [torch.empty_like(local) for _ in range(self.world_size)]
        dist.all_gather(parts, local)
        return torch.stack(parts).cpu()

    def state_dict(self) -> dict[str, object]:
        """Collective when world_size > 1: every rank returns the same whole table (a checkpoint writer that drops
        replicated tensors then keeps all ranks' rows)."""
        states = self._gather_rank_states()
        return {"version": _i64([STATE_VERSION]), "seed_namespace_version": _i64([SEED_NAMESPACE_VERSION]),
                "seed_base": _i64([_signed(self._seed_base)]), "subsequence_stride": _i64([SUBSEQUENCE_STRIDE]),
                "world_size": _i64([self.world_size]), "rank_ids": torch.arange(self.world_size, dtype=torch.int64),
                "logical_keys": list(self.logical_keys), "states": states.to(torch.int64).clone()}

    def load_state_dict(self, state_dict: Mapping[str, object]) -> None:
        if set(state_dict) != _V2_FIELDS:
            raise RuntimeError(f"invalid localCTA SR checkpoint fields: expected={sorted(_V2_FIELDS)}, "
                               f"got={sorted(state_dict)}")
        version = _scalar("version", state_dict["version"])
        namespace = _scalar("seed_namespace_version", state_dict["seed_namespace_version"])
        seed_base = _scalar("seed_base", state_dict["seed_base"]) & UINT64_MAX
        stride = _scalar("subsequence_stride", state_dict["subsequence_stride"])
        world = _scalar("world_size", state_dict["world_size"])
        if version != STATE_VERSION:
            raise RuntimeError(f"unsupported localCTA SR checkpoint version {version}; expected {STATE_VERSION}")
        if namespace != SEED_NAMESPACE_VERSION:
            raise RuntimeError(f"unsupported localCTA SR seed namespace version {namespace}; expected "
                               f"{SEED_NAMESPACE_VERSION}")
        if stride != SUBSEQUENCE_STRIDE:
            raise RuntimeError(f"localCTA SR checkpoint stride {stride} does not match runtime stride "
                               f"{SUBSEQUENCE_STRIDE}")
        if world != self.world_size:
            raise RuntimeError("localCTA SR checkpoint world_size differs from the runtime; refusing to remap rank "
                               f"stochastic streams: checkpoint={world}, runtime={self.world_size}")
        if not torch.equal(_field("rank_ids", state_dict["rank_ids"]), torch.arange(self.world_size, dtype=torch.int64)):
            raise RuntimeError("localCTA SR checkpoint rank namespace is malformed; refusing to remap stochastic streams")
        if tuple(state_dict["logical_keys"]) != self.logical_keys:
            raise RuntimeError("localCTA SR logical-producer manifest differs from the checkpoint; refusing to remap "
                               "stochastic subsequences")
        states = _field("states", state_dict["states"])
        shape = (self.world_size, len(self.logical_keys), 2)
        if tuple(states.shape) != shape:
            raise RuntimeError(f"invalid localCTA SR state matrix shape: expected {shape}, got {tuple(states.shape)}")
        for r in range(self.world_size):
            for s in range(len(self.logical_keys)):
                if int(states[r, s, 0]) != _signed(self._seed_for(seed_base, r, s)):
                    raise RuntimeError(f"localCTA SR checkpoint seed namespace is inconsistent at rank={r}, slot={s}; "
                                       "refusing resume")
        self._seed_base = seed_base
        self._write_rows(states[self.rank])

    def migrate_from_v1_state_dict(self, state_dict: Mapping[str, object]) -> None:
        """The older format held ONE table [n_keys, 2] with seeds ``base + slot + 1`` on every rank.  Its counters are
        taken as they are for every rank; rank 0 keeps its seeds, the other ranks move to their own (so the resume is
        not bit-continuous there).  Only on the operator's explicit request (register_with_checkpointer)."""
        if set(state_dict) != _V1_FIELDS:
            raise RuntimeError(f"invalid localCTA SR v1 checkpoint fields: expected={sorted(_V1_FIELDS)}, "
                               f"got={sorted(state_dict)}")
        version = _scalar("version", state_dict["version"])
        stride = _scalar("subsequence_stride", state_dict["subsequence_stride"])
        if version != LEGACY_STATE_VERSION:
            raise RuntimeError(f"localCTA SR migration requires v1, got version {version}")
        if stride != SUBSEQUENCE_STRIDE:
            raise RuntimeError(f"localCTA SR v1 stride {stride} does not match runtime stride {SUBSEQUENCE_STRIDE}")
        if tuple(state_dict["logical_keys"]) != self.logical_keys:
            raise RuntimeError("localCTA SR v1 logical-producer manifest differs from the runtime; refusing migration")
        states = _field("states", state_dict["states"])
        shape = (len(self.logical_keys), 2)
        if tuple(states.shape) != shape:
            raise RuntimeError(f"invalid localCTA SR v1 state matrix shape: expected {shape}, got {tuple(states.shape)}")
        seed_base = ((int(states[0, 0]) & UINT64_MAX) - 1) & UINT64_MAX
        for s in range(len(self.logical_keys)):
            if int(states[s, 0]) != _signed(seed_base + s + 1):
                raise RuntimeError("localCTA SR v1 seed slots are inconsistent; refusing migration")
        self._seed_base = seed_base
        self._write_rows(self._fresh_rows(seed_base, [int(states[s, 1]) for s in range(len(self.logical_keys))]))


# ---- the installed table -------------------------------------------------------------------------------------------

_ACTIVE: LocalCTASRState | None = None


def active_localcta_sr_state() -> LocalCTASRState | None:
    return _ACTIVE


def set_active_localcta_sr_state(state: LocalCTASRState | None) -> None:
    global _ACTIVE
    _ACTIVE = state


def get_localcta_sr_state(logical_key: str, device=None) -> torch.Tensor | None:
    return None if _ACTIVE is None else _ACTIVE.get(logical_key, device)


@contextmanager
def preserve_localcta_sr_state_during_cuda_graph_capture(logical_keys: Iterable[str]) -> Iterator[None]:
    if _ACTIVE is None:
        yield
    else:
        with _ACTIVE.preserve_during_cuda_graph_capture(logical_keys):
            yield


def build_localcta_sr_state_for_trainer(model_parts: Iterable[torch.nn.Module], *, device, training_steps: int,
                                        gradient_accumulation_steps: int) -> LocalCTASRState | None:
    """Reference :637-683.  Installs a table for the model's gradient producers when the environment asks for
    gradient SR on the localCTA-v4 route (seed and base from NVFP4_RNG_SEED / NVFP4_RNG_SUBSEQUENCE_BASE); refuses
    activation / weight SR (no checkpointed counter exists for them) and scale SR together with a QKV producer
    (that producer takes data SR only)."""
    set_active_localcta_sr_state(None)
    if _localcta_v4_enabled() and (_role_sr_enabled("activation") or _role_sr_enabled("weight")):
        raise RuntimeError("checkpointed localCTA-v4 SR currently supports gradient producers only; activation/weight "
                           "SR would fall back to an uncheckpointed extension-global atomic and is therefore rejected")
    if not localcta_v4_grad_sr_enabled():
        return None
    keys = discover_logical_keys(model_parts)
    if _role_scale_sr_enabled("grad") and any(k.endswith(":sr:qkv_grad") for k in keys):
        raise RuntimeError("checkpointed localCTA gradient scale SR is unsupported for the QKV split3 producer; "
                           "disable NVFP4_SCALE_SR_GRAD until that ABI forwards scale stochastic rounding")
    state = LocalCTASRState(keys, device=device, user_seed=int(os.environ.get("NVFP4_RNG_SEED", "0")),
                            user_subsequence_base=int(os.environ.get("NVFP4_RNG_SUBSEQUENCE_BASE", "0")),
                            training_steps=training_steps, gradient_accumulation_steps=gradient_accumulation_steps,
                            reservation_margin=int(os.environ.get("LBT_LOCALCTA_SR_RESERVATION_MARGIN",
                                                                  str(DEFAULT_RESERVATION_MARGIN))))
    set_active_localcta_sr_state(state)
    return state


# ---- distributed-checkpoint hooks ------------------------------------------------------------------------------------

def checkpoint_localcta_sr_state_schema(checkpoint_id: str) -> str:
    """"missing", "v1", "v2" or "unknown", from a torch.distributed.checkpoint directory's metadata alone: the
    complete field set of a format AND the rank of its ``states`` tensor (2 / 3) must both fit."""
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    entries = FileSystemReader(checkpoint_id).read_metadata().state_dict_metadata
    prefix = CHECKPOINT_KEY + "."
    fields = {k[len(prefix):] for k in entries if k.startswith(prefix)}
    if not fields:
        return "missing"
    states = entries.get(prefix + "states")
    if not isinstance(states, TensorStorageMetadata):
        return "unknown"
    if fields == _V1_FIELDS and len(states.size) == 2:
        return "v1"
    if fields == _V2_FIELDS and len(states.size) == 3:
        return "v2"
    return "unknown"


def checkpoint_contains_localcta_sr_state(checkpoint_id: str) -> bool:
    return checkpoint_localcta_sr_state_schema(checkpoint_id) != "missing"


class _LegacyV1LoadState:
    """Destination a distributed-checkpoint load fills with a v1 table on its way into migrate_from_v1_state_dict."""

    def __init__(self, logical_keys: tuple[str, ...]) -> None:
        self.logical_keys = logical_keys
        self.loaded_state_dict: dict[str, object] | None = None

    def state_dict(self) -> dict[str, object]:
        return {"version": torch.zeros(1, dtype=torch.int64), "subsequence_stride": torch.zeros(1, dtype=torch.int64),
                "logical_keys": list(self.logical_keys),
                "states": torch.empty((len(self.logical_keys), 2), dtype=torch.int64)}

    def load_state_dict(self, state_dict: Mapping[str, object]) -> None:
        self.loaded_state_dict = {k: (v.detach().cpu().clone() if torch.is_tensor(v) else v)
                                  for k, v in state_dict.items()}


def _v1_migration_world_size(state: LocalCTASRState) -> None:
    asked = os.environ.get(V1_MIGRATION_ENV, "").strip().lower()
    if asked != V1_RANK_NAMESPACE_MIGRATION:
        detail = f"unsupported value {asked!r} for {V1_MIGRATION_ENV}; " if asked else ""
        raise RuntimeError("localCTA SR checkpoint uses the rank-correlated v1 RNG namespace. Resume is rejected by "
                           f"default. {detail}Set {V1_MIGRATION_ENV}={V1_RANK_NAMESPACE_MIGRATION} to explicitly "
                           "preserve persisted subsequence counters while moving each rank into the v2 seed namespace. "
                           "This transition is not bitwise-continuous on ranks greater than zero and does not infer "
                           "state from the checkpoint step.")
    raw = os.environ.get(V1_EXPECTED_WORLD_SIZE_ENV, "").strip()
    if not raw:
        raise RuntimeError(f"localCTA SR v1 did not checkpoint world_size. Set {V1_EXPECTED_WORLD_SIZE_ENV} to the "
                           "verified legacy world size before migration; refusing to infer it.")
    try:
        world = int(raw)
    except ValueError as exc:
        raise RuntimeError(f"invalid {V1_EXPECTED_WORLD_SIZE_ENV}={raw!r}; expected a positive integer") from exc
    if world <= 0:
        raise RuntimeError(f"invalid {V1_EXPECTED_WORLD_SIZE_ENV}={raw!r}; expected a positive integer")
    if world != state.world_size:
        raise RuntimeError("operator-verified localCTA SR v1 world size differs from the live runtime; refusing to "
                           f"remap rank streams: verified_v1={world}, runtime={state.world_size}")


def register_with_checkpointer(checkpointer, state: LocalCTASRState, logger) -> None:
    """Adds the table to a TorchTitan-style checkpoint manager (``states`` dict, ``dcp_load`` method, optional
    ``ft_manager``) and wraps its load (reference :761-902): a checkpoint WITHOUT the table loads everything else and
    then starts a new SR phase at the configured base; a v1 table is refused unless the operator names the migration
    and the world size it was written with; an unrecognised layout is refused.  Nothing is ever inferred from the
    training step."""
    if getattr(checkpointer, "ft_manager", None) is not None:
        raise RuntimeError("checkpointed localCTA SR is not yet compatible with TorchFT replica checkpoints; disable "
                           "TorchFT or extend its state closure before enabling localCTA-v4 gradient SR")
    if CHECKPOINT_KEY in checkpointer.states:
        raise RuntimeError(f"duplicate checkpoint state {CHECKPOINT_KEY!r}")
    checkpointer.states[CHECKPOINT_KEY] = state
    inner_load = checkpointer.dcp_load

    def dcp_load(this, state_dict, checkpoint_id, from_hf, from_quantized):
        request, new_phase, legacy = state_dict, False, None
        if CHECKPOINT_KEY in state_dict and not from_hf:
            try:
                schema = checkpoint_localcta_sr_state_schema(checkpoint_id)
            except Exception as exc:
                raise RuntimeError("could not verify localCTA SR state in checkpoint metadata; refusing an ambiguous "
                                   "resume") from exc
            if schema == "missing":
                request = {k: v for k, v in state_dict.items() if k != CHECKPOINT_KEY}
                new_phase = True
            elif schema == "v1":
                _v1_migration_world_size(state)
                legacy = _LegacyV1LoadState(state.logical_keys)
                request = dict(state_dict)
                request[CHECKPOINT_KEY] = legacy
            elif schema != "v2":
                raise RuntimeError("unrecognized localCTA SR checkpoint metadata; refusing an ambiguous or partial "
                                   "state load")
        result = inner_load(request, checkpoint_id=checkpoint_id, from_hf=from_hf, from_quantized=from_quantized)
        if new_phase:   # only after the rest has loaded; a repeated load in one process must not keep advanced rows
            state.reset_to_configured_base()
            logger.warning("Checkpoint predates checkpointed localCTA SR state; starting an explicit new SR phase at "
                           "NVFP4_RNG_SUBSEQUENCE_BASE. This resume is not bitwise-continuous and no step-based "
                           "subsequence inference was performed.")
        if legacy is not None:
            if legacy.loaded_state_dict is None:
                raise RuntimeError("localCTA SR v1 migration loader was not populated by DCP; refusing resume")
            state.migrate_from_v1_state_dict(legacy.loaded_state_dict)
            logger.warning("Explicitly migrated localCTA SR v1 to the rank-namespaced v2 ABI for rank %d/%d. Persisted "
                           "next-subsequence counters were preserved exactly and applied to every rank; rank zero "
                           "retains its v1 seed and ranks greater than zero enter deterministic disjoint seed "
                           "streams. The operator-verified legacy world size was %d. This is not bitwise-continuous "
                           "on ranks greater than zero and no step-based phase inference was performed.",
                           state.rank, state.world_size, state.world_size)
        return result

    checkpointer.dcp_load = types.MethodType(dcp_load, checkpointer)
