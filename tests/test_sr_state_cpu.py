"""The checkpointable stochastic-rounding coordinates (mxfp4_sr_state): against values the reference's own
module produced here (tests/golden/mxfp4_sr_state_reference_golden.json, written by make_golden.py --which sr_state),
the refusals of load_state_dict, and the gathered checkpoint of two gloo ranks."""
import copy
import importlib
import json
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "mxfp4_sr_state_reference_golden.json")


def _mod():
    return importlib.import_module("mfu-fp4-training_b200.mxfp4_sr_state")


def _make(sr, gold, rank, world):
    return sr.MXFP4SRState(gold["keys"], device="cpu", user_seed=gold["seed"], user_subsequence_base=gold["subsequence_base"],
                           training_steps=10, gradient_accumulation_steps=2, rank=rank, world_size=world)


def test_keys_and_streams_match_the_reference_module():
    sr = _mod()
    gold = json.load(open(GOLD))
    n = gold["names"]
    assert [sr.ffn_deriv_grad_key(n[0]), sr.qkv_grad_key(n[1]), sr.wo_grad_key(n[1]), sr.ffn_w2_grad_key(n[2]),
            sr.linear_grad_key("head")] == gold["keys"]
    for label, rank, world in (("single", 0, 1), ("rank1_of_2", 1, 2)):
        run = gold["runs"][label]
        st = _make(sr, gold, rank, world)
        assert list(st.logical_keys) == run["sorted_keys"] and st.reservations_per_slot == run["reservations_per_slot"]
        assert [list(st.reserve(gold["keys"][i])) for i in gold["script"]] == run["reserved"]
        assert [list(st.peek(k)) for k in gold["keys"]] == run["peek"]
        assert st._local_rows().tolist() == run["local_rows"]
        if world == 1:
            sd = st.state_dict()
            assert set(sd) == set(run["state_dict"])
            for k, v in run["state_dict"].items():
                assert (sd[k].tolist() if torch.is_tensor(sd[k]) else sd[k]) == v, k
                if torch.is_tensor(sd[k]):
                    assert sd[k].dtype == torch.int64


def test_checkpoint_round_trip_resumes_the_streams():
    sr = _mod()
    gold = json.load(open(GOLD))
    a = _make(sr, gold, 0, 1)
    for i in gold["script"]:
        a.reserve(gold["keys"][i])
    sd = a.state_dict()
    b = _make(sr, gold, 0, 1)
    b.load_state_dict(sd)
    for k in gold["keys"]:
        assert b.peek(k) == a.peek(k)
        assert b.reserve(k) == a.reserve(k)
    b.reset_to_configured_base()
    assert b.peek(gold["keys"][0])[1] == gold["subsequence_base"]
    # a checkpoint written under another seed base carries that base with it
    other = sr.MXFP4SRState(gold["keys"], user_seed=77, user_subsequence_base=0, training_steps=1,
                            gradient_accumulation_steps=1)
    other.reserve(gold["keys"][2])
    b.load_state_dict(other.state_dict())
    assert b.peek(gold["keys"][2]) == other.peek(gold["keys"][2])


def test_load_refuses_what_would_remap_a_stream():
    sr = _mod()
    gold = json.load(open(GOLD))
    st = _make(sr, gold, 0, 1)
    good = st.state_dict()

    def broken(edit):
        sd = copy.deepcopy(good)
        edit(sd)
        with pytest.raises(RuntimeError):
            _make(sr, gold, 0, 1).load_state_dict(sd)

    broken(lambda d: d.pop("rank_ids"))
    broken(lambda d: d.__setitem__("version", torch.tensor([2], dtype=torch.int64)))
    broken(lambda d: d.__setitem__("subsequence_stride", torch.tensor([1 << 31], dtype=torch.int64)))
    broken(lambda d: d.__setitem__("world_size", torch.tensor([2], dtype=torch.int64)))
    broken(lambda d: d.__setitem__("logical_keys", d["logical_keys"][:-1] + ["x:sr:linear_grad"]))
    broken(lambda d: d["states"].__setitem__((0, 0, 0), 5))                      # seed not derived from the base
    broken(lambda d: d["states"].__setitem__((0, 1, 1), int(d["states"][0, 1, 1]) + 1))   # off the stride
    broken(lambda d: d["states"].__setitem__((0, 1, 1), 0))                      # before the base
    broken(lambda d: d.__setitem__("states", d["states"].to(torch.int32)))
    with pytest.raises(RuntimeError):
        st.reserve("unknown:sr:qkv_grad")
    with pytest.raises(ValueError):
        sr.MXFP4SRState([], user_seed=0, user_subsequence_base=0, training_steps=1, gradient_accumulation_steps=1)
    with pytest.raises(ValueError):
        sr.MXFP4SRState(["k"], user_seed=0, user_subsequence_base=(1 << 64) - 5, training_steps=1,
                        gradient_accumulation_steps=1)
    with pytest.raises(ValueError):
        sr.MXFP4SRState(["k"], user_seed=0, user_subsequence_base=0, training_steps=1, gradient_accumulation_steps=1,
                        rank=2, world_size=2)


def test_active_state_helpers():
    sr = _mod()
    sr.set_active_mxfp4_sr_state(None)
    with pytest.raises(RuntimeError):
        sr.reserve_mxfp4_sr("a:sr:qkv_grad")
    st = sr.MXFP4SRState(["a:sr:qkv_grad"], user_seed=3, user_subsequence_base=9, training_steps=0,
                         gradient_accumulation_steps=1)
    sr.set_active_mxfp4_sr_state(st)
    try:
        assert sr.active_mxfp4_sr_state() is st
        with pytest.raises(RuntimeError):
            sr.reserve_mxfp4_sr(None)
        assert sr.reserve_mxfp4_sr("a:sr:qkv_grad") == (4, 9)
        assert sr.reserve_mxfp4_sr("a:sr:qkv_grad") == (4, 9 + (1 << 32))
    finally:
        sr.set_active_mxfp4_sr_state(None)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sr = _mod()
        keys = ["l0:sr:qkv_grad", "l0:sr:wo_grad", "l1:sr:ffn_deriv_grad"]
        st = sr.MXFP4SRState(keys, user_seed=100, user_subsequence_base=1 << 32, training_steps=4,
                             gradient_accumulation_steps=1)
        for _ in range(rank + 1):              # the ranks advance differently
            st.reserve(keys[0])
        st.reserve(keys[2])
        sd = st.state_dict()                   # collective
        states = sd["states"]
        ok = tuple(states.shape) == (world, 3, 2)
        for r in range(world):
            for s in range(3):
                ok = ok and int(states[r, s, 0]) == 100 + r * 3 + s + 1
            ok = ok and int(states[r, 0, 1]) == (1 << 32) * (1 + r + 1)
            ok = ok and int(states[r, 1, 1]) == (1 << 32) and int(states[r, 2, 1]) == (1 << 32) * 2
        fresh = sr.MXFP4SRState(keys, user_seed=100, user_subsequence_base=1 << 32, training_steps=4,
                                gradient_accumulation_steps=1)
        fresh.load_state_dict(sd)              # every rank picks its own row
        ok = ok and fresh.peek(keys[0]) == st.peek(keys[0]) and fresh.peek(keys[0])[0] == 100 + rank * 3 + 1
        mismatch = False
        try:                                   # different producers on the two ranks: refused at construction
            sr.MXFP4SRState(keys[: 2 + rank], user_seed=1, user_subsequence_base=0, training_steps=1,
                            gradient_accumulation_steps=1)
        except RuntimeError:
            mismatch = True
        q.put((rank, bool(ok), mismatch))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_ranks_share_one_checkpoint_and_keep_their_own_streams():
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
    assert all(r[1] for r in res), "gathered checkpoint or its reload is wrong"
    assert all(r[2] for r in res), "ranks with different producer lists must be refused"
