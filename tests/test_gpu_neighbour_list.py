"""Cell-list kernel against the brute-force oracle: the canonically sorted edge set must be bit-exact."""
import numpy as np
import pytest
import torch

from tace_b200 import synth
from tace_b200.neighbour_list import get_neighborhood, neighbor_list_batch

pytestmark = pytest.mark.gpu


def check(structure, cutoff):
    from oracle.neighbour_list import canonical_sort, neighbour_list

    ref_i, ref_s = neighbour_list(structure["positions"], structure["cell"], structure["pbc"], cutoff)
    ei, es, _, _ = get_neighborhood(structure["positions"], cutoff, structure["pbc"], structure["cell"])
    ei, es = canonical_sort(ei, es)
    assert ei.shape == ref_i.shape, (ei.shape, ref_i.shape)
    assert np.array_equal(ei, ref_i) and np.array_equal(es, ref_s)
    return ei


def test_cubic_fcc():
    ei = check(synth.fcc_supercell(3, 3.61, 0.05, seed=0), 5.0)
    assert ei.shape[1] > 0


def test_triclinic_small_cells_with_self_images():
    for s in synth.random_crystals(6, seed=7, nmin=2, nmax=10):
        check(s, 6.0)


def test_unwrapped_positions():
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=1)
    rng = np.random.default_rng(0)
    s["positions"] = s["positions"] + rng.integers(-2, 3, size=(s["positions"].shape[0], 3)) @ s["cell"]
    check(s, 4.5)


def test_mixed_and_open_boundaries():
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=2)
    for pbc in [(True, True, False), (False, False, False), (True, False, False)]:
        t = synth.Structure(s)
        t["pbc"] = pbc
        check(t, 4.5)


def test_single_atom_and_no_neighbours():
    one = synth.Structure(positions=np.zeros((1, 3)), atomic_numbers=np.array([1]), cell=np.eye(3) * 4.0, pbc=(True,) * 3)
    ei = check(one, 6.0)  # only self images
    assert ei.shape[1] > 0 and (ei[0] == ei[1]).all()
    far = synth.Structure(positions=np.array([[0.0, 0, 0], [10.0, 0, 0]]), atomic_numbers=np.array([1, 1]),
                          cell=np.eye(3) * 40.0, pbc=(False,) * 3)
    assert check(far, 3.0).shape[1] == 0


def test_batch_matches_per_structure():
    structs = synth.random_crystals(5, seed=3, nmin=3, nmax=20)
    b = synth.collate(structs)
    dev = torch.device("cuda:0")
    ei, es = neighbor_list_batch(torch.tensor(b["positions"], device=dev), torch.tensor(b["lattice"], device=dev),
                                 torch.tensor(b["pbc"], device=dev), torch.tensor(b["ptr"], dtype=torch.int32, device=dev), 6.0)
    from oracle.neighbour_list import canonical_sort, neighbour_list
    ref_i, ref_s = [], []
    for s, off in zip(structs, b["ptr"][:-1]):
        a, c = neighbour_list(s["positions"], s["cell"], s["pbc"], 6.0)
        ref_i.append(a + off)
        ref_s.append(c)
    ref_i, ref_s = canonical_sort(np.concatenate(ref_i, 1), np.concatenate(ref_s, 0))
    gi, gs = canonical_sort(ei.cpu().numpy(), es.cpu().numpy())
    assert np.array_equal(gi, ref_i) and np.array_equal(gs, ref_s)
    # grouped by target: row 1 is non-decreasing
    assert (np.diff(ei[1].cpu().numpy()) >= 0).all()
