"""Spatial domain decomposition: grid choice, halo plans and the ghost exchange, checked on the CPU.

The edge set every rank derives from owned + ghost atoms must equal, taken together, the periodic
neighbour list of the whole system (the NL oracle); the two exchanges must be adjoint to each other.
Multi-rank runs use gloo with two and four ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.neighbour_list import neighbour_list
from tace_b200 import synth
from tace_b200.domain import Domain, DomainGrid, build_halo_plan, cell_heights, choose_grid


def test_choose_grid_minimises_block_surface():
    assert choose_grid(8, [10.0, 10.0, 10.0]) == (2, 2, 2)
    assert choose_grid(4, [10.0, 10.0, 40.0]) == (1, 1, 4)
    assert choose_grid(2, [30.0, 10.0, 10.0]) == (2, 1, 1)
    assert choose_grid(1, [1.0, 2.0, 3.0]) == (1, 1, 1)
    g = choose_grid(6, [10.0, 10.0, 10.0])
    assert g[0] * g[1] * g[2] == 6
    # sheared cell: the height along a is the distance between the planes spanned by b and c
    h = cell_heights(np.array([[4.0, 0, 0], [2.0, 3.0, 0], [0, 0, 5.0]]))
    assert np.allclose(h, [4.0 * 3.0 / np.hypot(2.0, 3.0), 3.0, 5.0])


def _global_edges(structure, cutoff):
    ei, sh = neighbour_list(structure["positions"], structure["cell"], (True, True, True), cutoff)
    vec = structure["positions"][ei[1]] - structure["positions"][ei[0]] + sh @ structure["cell"]
    return ei, vec


def _edge_keys(target_ids, source_ids, vec):
    """Multiset key of an edge: ids plus the vector rounded to 1e-6 (images of one pair differ by a cell vector)."""
    q = np.round(vec * 1e6).astype(np.int64)
    rows = np.concatenate([np.asarray(target_ids)[:, None], np.asarray(source_ids)[:, None], q], axis=1)
    return sorted(map(tuple, rows.tolist()))


def _local_edges(pos_local, n_owned, cutoff):
    d = pos_local[:n_owned, None, :] - pos_local[None, :, :]  # target - source
    r2 = (d * d).sum(-1)
    t, s = np.nonzero(r2 < cutoff * cutoff)
    keep = t != s
    return t[keep], s[keep], d[t[keep], s[keep]]


@pytest.mark.parametrize("grid", [(1, 1, 1), (2, 1, 1), (2, 2, 1), (1, 2, 2), (2, 2, 2), (3, 1, 2)])
def test_plans_reproduce_the_periodic_edge_set(grid):
    s = synth.fcc_supercell(4, 3.61, 0.05, seed=3)
    _check_plans(s["positions"], s["cell"], grid, 4.0, 0.4)


@pytest.mark.parametrize("grid", [(2, 1, 1), (4, 1, 1), (2, 2, 1)])
def test_plans_with_blocks_of_vacuum(grid):
    """A slab in a long box: some blocks own no atom (and may or may not see ghosts).  Their plans must still pair up
    with their neighbours' and the union of the local edge lists must stay the periodic neighbour list."""
    s = synth.fcc_supercell(3, 3.61, 0.05, seed=3)
    cell = s["cell"].copy()
    cell[0, 0] *= 3.0  # the atoms fill about a third of the box along x, away from the cell boundary
    pos = s["positions"] + np.array([1.0, 0.0, 0.0])
    plans = _check_plans(pos, cell, grid, 4.0, 0.4)
    assert any(p.n_owned == 0 for p in plans)
    assert any(p.n_owned == 0 and p.n_ghost > 0 for p in plans) or grid[0] > 2


def _check_plans(pos, cell, grid, cutoff, skin):
    dg = DomainGrid(grid)
    W = dg.world_size
    inv = np.linalg.inv(cell)
    frac = pos @ inv
    frac -= np.floor(frac)
    frac_t = torch.tensor(frac)
    owner = dg.owner_of(frac_t).numpy()
    rows = [np.nonzero(owner == r)[0] for r in range(W)]
    frac_by_rank = [frac_t[r] for r in rows]
    gw = (cutoff + skin) / cell_heights(cell)
    plans = [build_halo_plan(dg, r, frac_by_rank, gw) for r in range(W)]
    # both sides of every message agree
    for r in range(W):
        for q in plans[r].peers:
            off, cnt = plans[q].recv_slice.get(r, (0, 0))
            assert plans[r].send_index[q].numel() == cnt
            if cnt:
                assert torch.equal(plans[q].ghost_owner_index[off:off + cnt], plans[r].send_index[q])
                assert (plans[q].ghost_owner[off:off + cnt] == r).all()
            assert sum(c for _, c in plans[r].send_parts[q]) == plans[r].send_index[q].numel()
    # union of the local edge lists == periodic neighbour list of the whole system
    wrapped = frac @ cell
    keys = []
    for r in range(W):
        p = plans[r]
        gid = np.concatenate([rows[r]] + [rows[int(o)][[int(i)]] for o, i in zip(p.ghost_owner, p.ghost_owner_index)]) \
            if p.n_ghost else rows[r]
        gpos = wrapped[gid[p.n_owned:]] + p.ghost_shift.numpy().astype(np.float64) @ cell
        local = np.concatenate([wrapped[rows[r]], gpos]) if p.n_ghost else wrapped[rows[r]]
        t, srcs, d = _local_edges(local, p.n_owned, cutoff)
        keys += _edge_keys(gid[t], gid[srcs], d)
    ei, vec = _global_edges({"positions": wrapped, "cell": cell}, cutoff)
    assert sorted(keys) == _edge_keys(ei[1], ei[0], vec)
    return plans


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        s = synth.fcc_supercell(4, 3.61, 0.05, seed=5, species=(13, 29), fractions=(0.3, 0.7))
        pos, cell, z = s["positions"], s["cell"], s["atomic_numbers"]
        n = len(pos)
        cutoff, skin = 4.0, 0.4
        dom = Domain(cell, cutoff, skin, rank, world, torch.device("cpu"))
        lo, hi = (n * rank) // world, (n * (rank + 1)) // world
        state = {"positions": torch.tensor(pos[lo:hi]), "ids": torch.arange(lo, hi), "z": torch.tensor(np.asarray(z)[lo:hi])}
        new = dom.partition(state)
        ok = True
        # every atom has exactly one owner and its payload travelled with it
        counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([dom.n_owned]))
        ok &= sum(int(c) for c in counts) == n
        ok &= bool((new["z"].numpy() == np.asarray(z)[new["ids"].numpy()]).all())
        # ghost positions = image-translated owner positions; ghost payload = owner payload
        local_pos = dom.local_positions(new["positions"])
        local_ids = dom.local_rows(new["ids"])
        frac = pos @ np.linalg.inv(cell)
        wrapped = (frac - np.floor(frac)) @ cell
        expect = wrapped[local_ids.numpy()]
        expect[dom.n_owned:] += dom.plan.ghost_shift.numpy().astype(np.float64) @ cell
        ok &= bool(np.allclose(local_pos.numpy(), expect, atol=1e-12))
        # local edges, all ranks together, are the periodic neighbour list
        t, srcs, d = _local_edges(local_pos.numpy(), dom.n_owned, cutoff)
        gid = local_ids.numpy()
        mine = _edge_keys(gid[t], gid[srcs], d)
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        ei, vec = _global_edges({"positions": wrapped, "cell": cell}, cutoff)
        ok &= sorted(k for part in everyone for k in part) == _edge_keys(ei[1], ei[0], vec)
        # adjointness: <forward(x), y> summed over ranks == <x, reverse(y)> on owned rows
        g = torch.Generator().manual_seed(100 + rank)
        total = dom.n_owned + dom.n_ghost
        x = torch.zeros(total, 5, dtype=torch.float64)
        x[: dom.n_owned] = torch.randn(dom.n_owned, 5, generator=g, dtype=torch.float64)
        y = torch.randn(total, 5, generator=g, dtype=torch.float64)
        fx = torch.empty_like(x)
        dom.exchange.forward_exchange(x, fx, 5)
        ry = torch.empty_like(y)
        dom.exchange.reverse_exchange(y, ry, 5)
        lhs = (fx * y).sum().reshape(1)
        rhs = (x[: dom.n_owned] * ry[: dom.n_owned]).sum().reshape(1)
        dist.all_reduce(lhs)
        dist.all_reduce(rhs)
        ok &= bool(torch.allclose(lhs, rhs, rtol=1e-12))
        ok &= bool(torch.equal(ry[dom.n_owned:], y[dom.n_owned:]))
        # a displaced atom triggers a new partition on every rank
        moved = new["positions"].clone()
        ok &= not dom.needs_partition(moved)
        if rank == 0:
            moved[0, 0] += 0.6 * skin
        ok &= dom.needs_partition(moved)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_exchange_ghosts(world):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert all(ret[r] for r in range(world))


def test_halo_wider_than_cell_is_rejected():
    dg = DomainGrid((1, 1, 1))
    with pytest.raises(ValueError):
        build_halo_plan(dg, 0, [torch.rand(4, 3, dtype=torch.float64)], [1.2, 0.3, 0.3])
