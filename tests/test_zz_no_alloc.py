"""The allocation-free neighbour-list entry point against the regular count + fill pair.

Some hosts cannot let a plugin allocate device memory while they run (an MD engine that owns the whole
GPU through its own pool, or a loop that cannot take the synchronisation a cudaMalloc implies), so
``tace_nl_build_noalloc`` works out of a fixed array inside the library.  Its edges must be identical to
the regular entry points', on two calls in a row (the second call reuses the array the first one used).
Collected last on purpose: a failure here cannot hide any other test under ``-x``.
"""
import ctypes

import numpy as np
import pytest
import torch

from tace_b200 import lib as _lib
from tace_b200 import synth
from tace_b200.neighbour_list import neighbor_list_batch

pytestmark = pytest.mark.gpu


def build_noalloc(pos, lat, pbc, ptr, cutoff, max_edges):
    lib = _lib.load()
    dev = pos.device
    n = pos.shape[0]
    row_ptr = torch.full((n + 1,), -1, dtype=torch.int64, device=dev)
    edge_index = torch.full((2, max_edges), -1, dtype=torch.int64, device=dev)
    shifts = torch.full((max_edges, 3), 99, dtype=torch.int32, device=dev)
    st = lib.tace_nl_build_noalloc(pos.data_ptr(), lat.data_ptr(), pbc.data_ptr(), ptr.data_ptr(), lat.shape[0], n, float(cutoff),
                                   max_edges, row_ptr.data_ptr(), edge_index.data_ptr(), shifts.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream)
    return st, row_ptr, edge_index, shifts


def inputs(structs, dev):
    b = synth.collate(structs)
    return (torch.tensor(b["positions"], device=dev), torch.tensor(b["lattice"], device=dev),
            torch.tensor(b["pbc"], device=dev), torch.tensor(b["ptr"], dtype=torch.int32, device=dev))


def test_matches_regular_entry_points_twice_in_a_row():
    dev = torch.device("cuda:0")
    cases = [synth.random_crystals(5, seed=3, nmin=3, nmax=20), [synth.fcc_supercell(3, 3.61, 0.05, seed=0)]]
    for repeat in range(2):            # second round runs on scratch left behind by the first
        for structs in cases:
            pos, lat, pbc, ptr = inputs(structs, dev)
            ref_ei, ref_es = neighbor_list_batch(pos, lat, pbc, ptr, 6.0)
            E = ref_ei.shape[1]
            st, row_ptr, ei, es = build_noalloc(pos, lat, pbc, ptr, 6.0, E + 7)
            assert st == 0
            torch.cuda.synchronize()
            assert int(row_ptr[-1]) == E and int(row_ptr[0]) == 0
            counts = torch.bincount(ref_ei[1], minlength=pos.shape[0])
            assert torch.equal(row_ptr[1:] - row_ptr[:-1], counts)
            assert torch.equal(ei[:, :E], ref_ei) and torch.equal(es[:E], ref_es)
            assert (ei[:, E:] == -1).all() and (es[E:] == 99).all()   # nothing written past the edges found


def test_capacity_limits_and_truncation():
    dev = torch.device("cuda:0")
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0)
    pos, lat, pbc, ptr = inputs([s], dev)
    ref_ei, _ = neighbor_list_batch(pos, lat, pbc, ptr, 5.0)
    E = ref_ei.shape[1]
    st, row_ptr, ei, es = build_noalloc(pos, lat, pbc, ptr, 5.0, E // 2)   # too small: count still reported
    assert st == 0
    torch.cuda.synchronize()
    assert int(row_ptr[-1]) == E and torch.equal(ei[:, : E // 2], ref_ei[:, : E // 2])
    big = torch.zeros(16385, 3, dtype=torch.float64, device=dev)
    bptr = torch.tensor([0, 16385], dtype=torch.int32, device=dev)
    st, *_ = build_noalloc(big, lat, pbc, bptr, 5.0, 8)
    assert st == -3 and b"capacity" in _lib.load().tace_status_string(st)
