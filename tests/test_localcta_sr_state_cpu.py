"""The per-producer checkpointable stochastic-rounding table (localcta_sr_state): against values the reference's own
module produced here (tests/golden/localcta_sr_state_reference_golden.json, written by make_golden.py --which
localcta_sr_state), the refusals of its loaders, the distributed-checkpoint hooks, and the gathered checkpoint of two
gloo ranks.  The consumer's advance (``state[1] += launches * 2**32`` on the device) is done by hand on CPU rows."""
import copy
import importlib
import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = json.load(open(os.path.join(ROOT, "tests", "golden", "localcta_sr_state_reference_golden.json")))


def _mod():
    return importlib.import_module("mfu-fp4-training_b200.localcta_sr_state")


def _make(sr, rank=0, world=1, keys=None, seed=None, base=None, **kw):
    return sr.LocalCTASRState(GOLD["keys"] if keys is None else keys, device="cpu",
                              user_seed=GOLD["seed"] if seed is None else seed,
                              user_subsequence_base=GOLD["subsequence_base"] if base is None else base,
                              training_steps=kw.pop("training_steps", 10), gradient_accumulation_steps=2, rank=rank,
                              world_size=world, **kw)


def _play(sr, st):
    for i, n in GOLD["script"]:
        st.get(GOLD["keys"][i])[1] += n * sr.SUBSEQUENCE_STRIDE


def test_keys_rows_and_checkpoint_match_the_reference_module():
    sr = _mod()
    n = GOLD["names"]
    assert [sr.ffn_deriv_grad_key(n[0]), sr.qkv_grad_key(n[1]), sr.wo_grad_key(n[1]), sr.ffn_w2_grad_key(n[2])] == GOLD["keys"]
    for label, rank, world in (("single", 0, 1), ("rank1_of_2", 1, 2)):
        run = GOLD["runs"][label]
        st = _make(sr, rank, world)
        assert list(st.logical_keys) == run["sorted_keys"] and st.reservations_per_slot == run["reservations_per_slot"]
        assert st._local_state_matrix().tolist() == run["initial_rows"]
        _play(sr, st)
        assert st._local_state_matrix().tolist() == run["rows_after_script"]
        if world == 1:
            sd = st.state_dict()
            assert set(sd) == set(run["state_dict"])
            for k, v in run["state_dict"].items():
                assert (sd[k].tolist() if torch.is_tensor(sd[k]) else sd[k]) == v, k
                if torch.is_tensor(sd[k]):
                    assert sd[k].dtype == torch.int64


def test_rows_are_views_of_one_table_and_seeds_are_unique_over_ranks_and_producers():
    sr = _mod()
    st = _make(sr)
    row = st.get(GOLD["keys"][0])
    assert row.shape == (2,) and row.dtype == torch.int64
    assert row.untyped_storage().data_ptr() == st._local_state_matrix().untyped_storage().data_ptr()
    seeds = set()
    for rank in range(4):
        rows = _make(sr, rank, 4, seed=100)._local_state_matrix()
        seeds.update(int(s) for s in rows[:, 0])
    assert len(seeds) == 4 * len(GOLD["keys"])
    with pytest.raises(RuntimeError, match="unregistered localCTA SR logical identity"):
        st.get("nobody:sr:wo_grad")
    with pytest.raises(RuntimeError, match="but its producer is on"):
        st.get(GOLD["keys"][0], device="meta")


@pytest.mark.parametrize("rank,world,err", [(0, 0, "world_size must be positive"), (-1, 2, r"rank must be in \[0, world_size\)"),
                                            (2, 2, r"rank must be in \[0, world_size\)")])
def test_bad_rank_namespace_is_refused(rank, world, err):
    with pytest.raises(ValueError, match=err):
        _make(_mod(), rank, world)


def test_construction_refusals_and_uint64_wrap():
    sr = _mod()
    with pytest.raises(ValueError, match="at least one logical producer"):
        _make(sr, keys=[])
    with pytest.raises(RuntimeError, match="non-empty stable _lbt_debug_name"):
        sr.qkv_grad_key("")
    with pytest.raises(ValueError, match="insufficient uint64 headroom"):
        _make(sr, base=sr.UINT64_MAX - 10)
    with pytest.raises(ValueError, match=r"must be in \[0, 2\*\*64 - 1\]"):
        _make(sr, seed=1 << 64)
    with pytest.raises(ValueError, match="gradient_accumulation_steps must be positive"):
        sr.LocalCTASRState(["a"], device="cpu", user_seed=0, user_subsequence_base=0, training_steps=1,
                           gradient_accumulation_steps=0)
    st = _make(sr, keys=["a", "b"], seed=sr.UINT64_MAX, base=0)   # seeds wrap to 0 and 1, stored as signed words
    assert st._local_state_matrix()[:, 0].tolist() == [0, 1]
    st = _make(sr, keys=["a"], seed=(1 << 63) - 1, base=0)
    assert st.get("a")[0].item() == -(1 << 63)


def test_checkpoint_round_trip_resumes_and_the_snapshot_does_not_alias():
    sr = _mod()
    a = _make(sr)
    _play(sr, a)
    sd = a.state_dict()
    snap = sd["states"].clone()
    a.get(GOLD["keys"][0])[1] += sr.SUBSEQUENCE_STRIDE
    assert torch.equal(sd["states"], snap)
    b = _make(sr, seed=5, base=9 << 32)   # other configured seed / base: the checkpoint's win
    b.load_state_dict(sd)
    assert b._local_state_matrix().tolist() == GOLD["runs"]["single"]["rows_after_script"]
    assert b.state_dict()["seed_base"].tolist() == sd["seed_base"].tolist()
    b.reset_to_configured_base()
    assert b._local_state_matrix().tolist() == _make(sr, seed=5, base=9 << 32)._local_state_matrix().tolist()


def test_load_refuses_what_would_remap_a_stream():
    sr = _mod()
    a = _make(sr)
    sd = a.state_dict()

    def broken(**kw):
        d = copy.deepcopy(sd)
        d.update(kw)
        return d

    cases = [(broken(version=torch.tensor([3])), "unsupported localCTA SR checkpoint version"),
             (broken(seed_namespace_version=torch.tensor([2])), "unsupported localCTA SR seed namespace version"),
             (broken(subsequence_stride=torch.tensor([1 << 31])), "does not match runtime stride"),
             (broken(world_size=torch.tensor([2])), "world_size differs from the runtime"),
             (broken(rank_ids=torch.tensor([1])), "rank namespace is malformed"),
             (broken(logical_keys=list(reversed(sd["logical_keys"]))), "manifest differs from the checkpoint"),
             (broken(states=sd["states"][:, :2]), "invalid localCTA SR state matrix shape"),
             (broken(states=sd["states"].to(torch.int32)), "must be an int64 tensor"),
             (broken(seed_base=torch.tensor([7])), "seed namespace is inconsistent"),
             (broken(version=torch.tensor([2, 2])), "must contain one value")]
    extra = copy.deepcopy(sd)
    extra["more"] = torch.zeros(1, dtype=torch.int64)
    cases.append((extra, "invalid localCTA SR checkpoint fields"))
    for d, msg in cases:
        with pytest.raises(RuntimeError, match=msg):
            _make(sr).load_state_dict(d)
    with pytest.raises(RuntimeError, match="require an initialized distributed process group"):
        _make(sr, 1, 2).state_dict()


def test_v1_migration_keeps_counters_and_moves_other_ranks_to_their_own_seeds():
    sr = _mod()
    v1 = GOLD["v1"]["state_dict"]

    def payload():
        return {"version": torch.tensor(v1["version"]), "subsequence_stride": torch.tensor(v1["subsequence_stride"]),
                "logical_keys": list(v1["logical_keys"]), "states": torch.tensor(v1["states"], dtype=torch.int64)}

    for rank in (0, 1):
        st = _make(sr, rank, 2)
        st.migrate_from_v1_state_dict(payload())
        assert st._local_state_matrix().tolist() == GOLD["v1"]["rows"][str(rank)]
    bad = payload()
    bad["states"][2, 0] += 1
    with pytest.raises(RuntimeError, match="v1 seed slots are inconsistent"):
        _make(sr).migrate_from_v1_state_dict(bad)
    bad = payload()
    bad["version"] = torch.tensor([2])
    with pytest.raises(RuntimeError, match="migration requires v1"):
        _make(sr).migrate_from_v1_state_dict(bad)
    bad = payload()
    bad["world_size"] = torch.tensor([1])
    with pytest.raises(RuntimeError, match="invalid localCTA SR v1 checkpoint fields"):
        _make(sr).migrate_from_v1_state_dict(bad)


def test_capture_preservation_rolls_back_only_what_ran_inside():
    sr = _mod()
    st = _make(sr, keys=["a", "b"], seed=41, base=17)
    before = st.get("a").clone()
    with st.preserve_during_cuda_graph_capture(("a", "a")):
        st.get("a")[1] += 4 * sr.SUBSEQUENCE_STRIDE
        st.get("b")[1] += sr.SUBSEQUENCE_STRIDE
    assert torch.equal(st.get("a"), before)
    assert st.get("b").tolist() == [43, 17 + sr.SUBSEQUENCE_STRIDE]   # not named: kept
    with st.preserve_during_cuda_graph_capture(()):
        st.get("a")[1] += sr.SUBSEQUENCE_STRIDE
    assert st.get("a").tolist() == [42, 17 + sr.SUBSEQUENCE_STRIDE]
    with pytest.raises(RuntimeError, match="unregistered"):
        with st.preserve_during_cuda_graph_capture(("c",)):
            pass


def test_installed_table_helpers():
    sr = _mod()
    sr.set_active_localcta_sr_state(None)
    assert sr.active_localcta_sr_state() is None and sr.get_localcta_sr_state("a") is None
    with sr.preserve_localcta_sr_state_during_cuda_graph_capture(("a",)):
        pass
    st = _make(sr, keys=["a"], seed=1, base=0)
    sr.set_active_localcta_sr_state(st)
    try:
        assert sr.active_localcta_sr_state() is st
        with sr.preserve_localcta_sr_state_during_cuda_graph_capture(("a",)):
            sr.get_localcta_sr_state("a")[1] += sr.SUBSEQUENCE_STRIDE
        assert sr.get_localcta_sr_state("a", "cpu").tolist() == [2, 0]
    finally:
        sr.set_active_localcta_sr_state(None)


_POLICY_ENV = ("USE_TK_LOCALCTA", "USE_TK_LOCALCTA_VARIANT", "NVFP4_USE_STOCHASTIC_ROUNDING", "NVFP4_SR_GRAD",
               "NVFP4_GRAD_SR_AXES", "NVFP4_USE_SCALE_STOCHASTIC_ROUNDING", "NVFP4_SCALE_SR_GRAD", "NVFP4_SR_ACTIVATION",
               "NVFP4_SCALE_SR_ACTIVATION", "NVFP4_SR_WEIGHT", "NVFP4_SCALE_SR_WEIGHT", "NVFP4_RNG_SEED",
               "NVFP4_RNG_SUBSEQUENCE_BASE", "LBT_LOCALCTA_SR_RESERVATION_MARGIN")


def _set_env(monkeypatch, env):
    for k in _POLICY_ENV:
        monkeypatch.delenv(k, raising=False)
    for k, v in env.items():
        monkeypatch.setenv(k, v)


def test_enable_policy_matches_the_reference_module(monkeypatch):
    sr = _mod()
    for case in GOLD["policy"]:
        _set_env(monkeypatch, case["env"])
        assert sr.localcta_v4_grad_sr_enabled() == case["grad_sr"], case["env"]
        for role, (any_sr, scale_sr) in case["role"].items():
            assert sr._role_sr_enabled(role) == any_sr and sr._role_scale_sr_enabled(role) == scale_sr, (case["env"], role)


def _stand_in(kind, name):
    m = type(kind, (torch.nn.Module,), {})()
    if name is not None:
        m._lbt_debug_name = name
    return m


def _model():
    root = torch.nn.Module()
    root.a = _stand_in("FusedAttentionFP4_TK", "layers.0.attention")
    root.b = _stand_in("FusedFeedForwardFP4_TK", "layers.0.feed_forward")
    root.c = _stand_in("FusedSquaredReLUFeedForwardFP4_TK", "layers.1.feed_forward")
    root.d = torch.nn.Linear(2, 2)
    return root


def test_discovery_and_the_trainer_hook(monkeypatch):
    sr = _mod()
    assert list(sr.discover_logical_keys([_model()])) == GOLD["discovered"]
    twin = _model()
    twin.e = _stand_in("FusedFeedForwardFP4_TK", "layers.0.feed_forward")
    with pytest.raises(RuntimeError, match="duplicate localCTA SR logical identity"):
        sr.discover_logical_keys([twin])
    nameless = torch.nn.Module()
    nameless.a = _stand_in("FusedFeedForwardFP4_TK", None)
    with pytest.raises(RuntimeError, match="non-empty stable _lbt_debug_name"):
        sr.discover_logical_keys([nameless])

    on = {"USE_TK_LOCALCTA": "1", "USE_TK_LOCALCTA_VARIANT": "v4"}
    try:
        _set_env(monkeypatch, {})
        assert sr.build_localcta_sr_state_for_trainer([_model()], device="cpu", training_steps=5,
                                                      gradient_accumulation_steps=1) is None
        _set_env(monkeypatch, dict(on, NVFP4_SR_GRAD="1", NVFP4_RNG_SEED="40", NVFP4_RNG_SUBSEQUENCE_BASE="16",
                                   LBT_LOCALCTA_SR_RESERVATION_MARGIN="3"))
        st = sr.build_localcta_sr_state_for_trainer([_model()], device="cpu", training_steps=5, gradient_accumulation_steps=2)
        assert sr.active_localcta_sr_state() is st and list(st.logical_keys) == GOLD["discovered"]
        assert st.reservations_per_slot == 6 * 2 + 3 and st.get(GOLD["discovered"][1]).tolist() == [42, 16]
        _set_env(monkeypatch, dict(on, NVFP4_SR_GRAD="1", NVFP4_SR_ACTIVATION="1"))
        with pytest.raises(RuntimeError, match="supports gradient producers only"):
            sr.build_localcta_sr_state_for_trainer([_model()], device="cpu", training_steps=5, gradient_accumulation_steps=1)
        assert sr.active_localcta_sr_state() is None
        _set_env(monkeypatch, dict(on, NVFP4_SR_GRAD="1", NVFP4_SCALE_SR_GRAD="1"))
        with pytest.raises(RuntimeError, match="unsupported for the QKV split3 producer"):
            sr.build_localcta_sr_state_for_trainer([_model()], device="cpu", training_steps=5, gradient_accumulation_steps=1)
        ffn_only = torch.nn.Module()
        ffn_only.b = _stand_in("FusedFeedForwardFP4_TK", "layers.0.feed_forward")
        assert sr.build_localcta_sr_state_for_trainer([ffn_only], device="cpu", training_steps=5,
                                                      gradient_accumulation_steps=1) is not None
    finally:
        sr.set_active_localcta_sr_state(None)


def _v1_table(sr, keys, seed_base=41, nxt=17):
    return {"version": torch.tensor([1]), "subsequence_stride": torch.tensor([sr.SUBSEQUENCE_STRIDE]),
            "logical_keys": sorted(keys), "states": torch.tensor([[seed_base + s + 1, nxt + s * sr.SUBSEQUENCE_STRIDE]
                                                                  for s in range(len(keys))], dtype=torch.int64)}


def test_distributed_checkpoint_round_trip_and_schema_classifier(tmp_path):
    import torch.distributed.checkpoint as dcp
    sr = _mod()
    keys = ["layer.0:sr:a", "layer.0:sr:b"]
    a = _make(sr, keys=keys, seed=41, base=17)
    a.get(keys[1])[1] += 5 * sr.SUBSEQUENCE_STRIDE
    path = str(tmp_path / "v2")
    dcp.save({sr.CHECKPOINT_KEY: a}, checkpoint_id=path)
    b = _make(sr, keys=keys, seed=999, base=999)
    dcp.load({sr.CHECKPOINT_KEY: b}, checkpoint_id=path)
    assert b._local_state_matrix().tolist() == a._local_state_matrix().tolist() == [[42, 17], [43, 17 + 5 * (1 << 32)]]
    assert sr.checkpoint_localcta_sr_state_schema(path) == "v2" and sr.checkpoint_contains_localcta_sr_state(path)

    path = str(tmp_path / "none")
    dcp.save({"other": torch.ones(1)}, checkpoint_id=path)
    assert sr.checkpoint_localcta_sr_state_schema(path) == "missing" and not sr.checkpoint_contains_localcta_sr_state(path)
    path = str(tmp_path / "v1")
    dcp.save({sr.CHECKPOINT_KEY: _v1_table(sr, keys)}, checkpoint_id=path)
    assert sr.checkpoint_localcta_sr_state_schema(path) == "v1"
    loader = sr._LegacyV1LoadState(tuple(keys))
    dcp.load({sr.CHECKPOINT_KEY: loader}, checkpoint_id=path)
    st = _make(sr, 1, 2, keys=keys, seed=0, base=0)
    st.migrate_from_v1_state_dict(loader.loaded_state_dict)
    assert st._local_state_matrix().tolist() == [[44, 17], [45, 17 + (1 << 32)]]
    path = str(tmp_path / "odd")
    odd = _v1_table(sr, keys)
    odd["unexpected"] = torch.ones(1)
    dcp.save({sr.CHECKPOINT_KEY: odd}, checkpoint_id=path)
    assert sr.checkpoint_localcta_sr_state_schema(path) == "unknown"


class _Manager:
    """What register_with_checkpointer needs of a checkpoint manager."""

    def __init__(self, v1_payload=None):
        self.states, self.ft_manager, self.seen, self.v1_payload = {}, None, None, v1_payload

    def dcp_load(self, state_dict, checkpoint_id, from_hf, from_quantized):
        self.seen = (state_dict, checkpoint_id, from_hf, from_quantized)
        if self.v1_payload is not None:
            state_dict["localcta_sr_state"].load_state_dict(self.v1_payload)
        return "loaded"


class _Log:
    def __init__(self):
        self.lines = []

    def warning(self, msg, *args):
        self.lines.append(msg % args if args else msg)


def test_checkpointer_hook_new_phase_v2_v1_and_refusals(monkeypatch):
    sr = _mod()
    keys = ["layer.0:sr:a", "layer.0:sr:b"]

    def fresh(rank=0, world=1):
        return _make(sr, rank, world, keys=keys, seed=41, base=17)

    # a checkpoint written before the table existed: everything else loads, then a new phase starts
    st, mgr, log = fresh(), _Manager(), _Log()
    monkeypatch.setattr(sr, "checkpoint_localcta_sr_state_schema", lambda _: "missing")
    sr.register_with_checkpointer(mgr, st, log)
    assert mgr.states[sr.CHECKPOINT_KEY] is st
    st.get(keys[0])[1] += 7 * sr.SUBSEQUENCE_STRIDE
    asked = {"other": object(), sr.CHECKPOINT_KEY: st}
    assert mgr.dcp_load(asked, "/old", False, False) == "loaded"
    assert sr.CHECKPOINT_KEY not in mgr.seen[0] and sr.CHECKPOINT_KEY in asked
    assert st._local_state_matrix().tolist() == [[42, 17], [43, 17]]
    assert "no step-based subsequence inference" in log.lines[0]
    with pytest.raises(RuntimeError, match="duplicate checkpoint state"):
        sr.register_with_checkpointer(mgr, st, log)

    # the current format goes through untouched; a load from another model format is not inspected at all
    st, mgr = fresh(), _Manager()
    monkeypatch.setattr(sr, "checkpoint_localcta_sr_state_schema", lambda _: "v2")
    sr.register_with_checkpointer(mgr, st, _Log())
    asked = {sr.CHECKPOINT_KEY: st}
    mgr.dcp_load(asked, "/new", False, False)
    assert mgr.seen[0][sr.CHECKPOINT_KEY] is st
    monkeypatch.setattr(sr, "checkpoint_localcta_sr_state_schema", lambda _: 1 / 0)
    mgr.dcp_load(asked, "/hf", True, False)
    assert mgr.seen[0] is asked
    with pytest.raises(RuntimeError, match="could not verify localCTA SR state"):
        mgr.dcp_load(asked, "/new", False, False)
    monkeypatch.setattr(sr, "checkpoint_localcta_sr_state_schema", lambda _: "unknown")
    with pytest.raises(RuntimeError, match="unrecognized localCTA SR checkpoint metadata"):
        mgr.dcp_load(asked, "/new", False, False)

    # the older format: only on request, and only with the world size it was written with
    monkeypatch.setattr(sr, "checkpoint_localcta_sr_state_schema", lambda _: "v1")
    st, mgr, log = fresh(1, 2), _Manager(_v1_table(sr, keys, nxt=17 + 3 * sr.SUBSEQUENCE_STRIDE)), _Log()
    sr.register_with_checkpointer(mgr, st, log)
    monkeypatch.delenv(sr.V1_MIGRATION_ENV, raising=False)
    monkeypatch.delenv(sr.V1_EXPECTED_WORLD_SIZE_ENV, raising=False)
    with pytest.raises(RuntimeError, match="Resume is rejected by default"):
        mgr.dcp_load({sr.CHECKPOINT_KEY: st}, "/v1", False, False)
    monkeypatch.setenv(sr.V1_MIGRATION_ENV, "guess")
    with pytest.raises(RuntimeError, match="unsupported value 'guess'"):
        mgr.dcp_load({sr.CHECKPOINT_KEY: st}, "/v1", False, False)
    monkeypatch.setenv(sr.V1_MIGRATION_ENV, sr.V1_RANK_NAMESPACE_MIGRATION)
    with pytest.raises(RuntimeError, match="did not checkpoint world_size"):
        mgr.dcp_load({sr.CHECKPOINT_KEY: st}, "/v1", False, False)
    for raw, msg in (("two", "expected a positive integer"), ("0", "expected a positive integer"),
                     ("4", "differs from the live runtime")):
        monkeypatch.setenv(sr.V1_EXPECTED_WORLD_SIZE_ENV, raw)
        with pytest.raises(RuntimeError, match=msg):
            mgr.dcp_load({sr.CHECKPOINT_KEY: st}, "/v1", False, False)
    assert st._local_state_matrix().tolist() == [[44, 17], [45, 17]]   # untouched by the refused loads
    monkeypatch.setenv(sr.V1_EXPECTED_WORLD_SIZE_ENV, "2")
    asked = {sr.CHECKPOINT_KEY: st}
    assert mgr.dcp_load(asked, "/v1", False, False) == "loaded"
    assert isinstance(mgr.seen[0][sr.CHECKPOINT_KEY], sr._LegacyV1LoadState) and asked[sr.CHECKPOINT_KEY] is st
    assert st._local_state_matrix().tolist() == [[44, 17 + 3 * (1 << 32)], [45, 17 + 4 * (1 << 32)]]
    assert "rank 1/2" in log.lines[0]

    mgr = _Manager()
    mgr.ft_manager = object()
    with pytest.raises(RuntimeError, match="not yet compatible with TorchFT"):
        sr.register_with_checkpointer(mgr, fresh(), _Log())


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_rank_worker(rank, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    try:
        sr = _mod()
        st = _make(sr, None, None)   # rank and world size from the process group
        assert (st.rank, st.world_size) == (rank, 2)
        for i, n in GOLD["script"][: 3 + 2 * rank]:
            st.get(GOLD["keys"][i])[1] += n * sr.SUBSEQUENCE_STRIDE
        sd = st.state_dict()
        assert tuple(sd["states"].shape) == (2, len(GOLD["keys"]), 2)
        assert torch.equal(sd["states"][rank], st._local_state_matrix())
        other = _make(sr, None, None, seed=1, base=0)
        other.load_state_dict(sd)
        assert torch.equal(other._local_state_matrix(), st._local_state_matrix())
        try:
            _make(sr, None, None, keys=GOLD["keys"][: 3 + rank])
            raise AssertionError("differing manifests were accepted")
        except RuntimeError as e:
            assert "manifests differ across ranks" in str(e)
        try:
            _make(sr, 0, 1)
            raise AssertionError("a namespace other than the process group's was accepted")
        except RuntimeError as e:
            assert "disagrees with the active process group" in str(e)
        if rank == 0:
            torch.save(sd["states"], out_path)
    finally:
        dist.destroy_process_group()


def test_two_ranks_share_one_checkpoint_and_keep_their_own_rows(tmp_path):
    out = str(tmp_path / "states.pt")
    mp.spawn(_two_rank_worker, args=(_free_port(), out), nprocs=2, join=True)
    states = torch.load(out)
    sr = _mod()
    for rank in (0, 1):
        st = _make(sr, rank, 2)
        for i, n in GOLD["script"][: 3 + 2 * rank]:
            st.get(GOLD["keys"][i])[1] += n * sr.SUBSEQUENCE_STRIDE
        assert states[rank].tolist() == st._local_state_matrix().tolist()
