"""Batch sharding across ranks: partition rule and result reassembly, run as two gloo ranks on the CPU
(the evaluation itself is a stand-in: the CUDA model cannot run here)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tace_b200 import synth
from tace_b200.shard import estimate_edges, evaluate_sharded, partition_lpt


def test_partition_is_balanced_and_complete():
    rng = np.random.default_rng(0)
    costs = rng.uniform(1.0, 100.0, size=64)
    for world in (1, 2, 4, 8):
        parts = partition_lpt(costs, world)
        assert sorted(i for p in parts for i in p) == list(range(64))
        loads = [sum(costs[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(costs)  # LPT bound
    assert partition_lpt([], 3) == [[], [], []]
    assert partition_lpt([5.0], 2) == [[0], []]


def test_edge_estimate_tracks_density():
    s = synth.fcc_supercell(3, 3.61, 0.0, seed=0)
    est = estimate_edges(s, 5.0) / len(s["positions"])
    assert 35.0 < est < 50.0  # 42 neighbours inside 5 A in FCC Cu


def _fake_eval(structs):
    return {"energy": np.array([float(s["positions"].sum()) for s in structs]),
            "stress": np.stack([np.eye(3) * len(s["positions"]) for s in structs]) if structs else np.zeros((0, 3, 3)),
            "forces": [s["positions"] * 2.0 for s in structs]}


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    structs = synth.random_crystals(9, seed=11, nmin=2, nmax=9)

    def gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    res = evaluate_sharded(structs, 6.0, _fake_eval, rank, world, gather)
    ref = _fake_eval(structs)
    ok = all(np.allclose(res["energy"][i], ref["energy"][i]) and np.allclose(res["forces"][i], ref["forces"][i])
             and np.allclose(res["stress"][i], ref["stress"][i]) for i in range(len(structs)))
    ret[rank] = ok
    dist.destroy_process_group()


def test_two_rank_gloo_roundtrip():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert ret[0] and ret[1]


def test_missing_rank_is_detected():
    structs = synth.random_crystals(4, seed=2, nmin=2, nmax=5)
    try:
        evaluate_sharded(structs, 6.0, _fake_eval, 0, 2, lambda obj: [obj])  # rank 1 never reports
    except RuntimeError as e:
        assert "did not report" in str(e)
    else:
        raise AssertionError("a dropped rank must raise")
