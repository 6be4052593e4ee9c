"""ASE calculator and LAMMPS ML-IAP entry points, driven with stand-in `atoms` / `data` objects."""
import numpy as np
import pytest
import torch

from tace_b200 import synth
from tace_b200.interface import TACEAseCalc, TACELammpsCalc
from tace_b200.interface.ase_calculator import export_tace
from helpers import make_models, oracle_batch, to_device

pytestmark = pytest.mark.gpu


class FakeAtoms:
    def __init__(self, s):
        self.s = s
        self.info = {}

    def get_positions(self): return self.s["positions"]
    def get_atomic_numbers(self): return self.s["atomic_numbers"]
    def get_cell(self): return self.s["cell"]
    def get_pbc(self): return np.array(self.s["pbc"])
    def __len__(self): return len(self.s["positions"])


def test_ase_calculator_matches_oracle_and_pt_roundtrip(tmp_path):
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0, species=(13, 29), fractions=(0.5, 0.5))
    model, oracle, cfg = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64)
    path = str(tmp_path / "model.pt")
    export_tace(model, path)
    calc = TACEAseCalc(path, device="cuda:0")
    calc.calculate(FakeAtoms(s))
    ref = oracle(oracle_batch([s], [13, 29], 4.0, torch.float64))
    assert abs(calc.results["energy"] - ref["energy"].item()) < 1e-8 * len(s["positions"])
    assert calc.results["free_energy"] == calc.results["energy"]
    assert np.abs(calc.results["forces"] - ref["forces"].numpy()).max() < 1e-7
    assert calc.results["stress"].shape == (3, 3)
    assert np.abs(calc.results["stress"] - ref["stress"][0].numpy()).max() < 1e-7
    assert set(calc.implemented_properties) >= {"energy", "free_energy", "forces", "stress"}


class FakeLammpsData:
    """Single-rank stand-in for the Kokkos ML-IAP data object: local atoms plus periodic ghost copies."""

    def __init__(self, s, cutoff, elements, device):
        from oracle.neighbour_list import neighbour_list
        ei, es = neighbour_list(s["positions"], s["cell"], s["pbc"], cutoff)
        n = len(s["positions"])
        ghost_of = {}          # (owner, shift) -> ghost index
        owners = []
        pair_i, pair_j, rij = [], [], []
        for (src, dst), sh in zip(ei.T, es):
            # edge source -> target with vector r_dst - r_src + sh @ cell; LAMMPS pair (i = target, j = source or its ghost)
            key = (int(src), tuple(int(v) for v in -sh))
            if key[1] == (0, 0, 0):
                j = int(src)
            else:
                if key not in ghost_of:
                    ghost_of[key] = n + len(owners)
                    owners.append(int(src))
                j = ghost_of[key]
            pair_i.append(int(dst)); pair_j.append(j)
            rij.append(s["positions"][dst] - s["positions"][src] + sh @ s["cell"])
        zs = sorted(elements)
        species = [zs.index(int(z)) for z in s["atomic_numbers"]]
        self.nlocal, self.ntotal, self.npairs = n, n + len(owners), len(pair_i)
        self.owner = torch.tensor(owners, dtype=torch.int64, device=device)
        self.elems = torch.tensor(species + [species[o] for o in owners], dtype=torch.int32, device=device)
        self.rij = torch.tensor(np.array(rij), dtype=torch.float64, device=device)
        self.pair_i = torch.tensor(pair_i, dtype=torch.int32, device=device)
        self.pair_j = torch.tensor(pair_j, dtype=torch.int32, device=device)
        self.eatoms = torch.zeros(n, dtype=torch.float64, device=device)
        self.energy = None
        self.pair_forces = None
        self.exchanges = 0

    def forward_exchange(self, src, dst, vec_len):
        dst.copy_(src)
        dst[self.nlocal:] = src[self.owner]
        self.exchanges += 1

    def reverse_exchange(self, src, dst, vec_len):
        dst.copy_(src)
        dst[: self.nlocal].index_add_(0, self.owner, src[self.nlocal:])
        self.exchanges += 1

    def update_pair_forces(self, f):
        self.pair_forces = f.clone()


@pytest.mark.parametrize("num_layers", [1, 2, 3])
def test_lammps_mliap_with_ghost_exchange_matches_graph_mode(num_layers):
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=4, species=(13, 29), fractions=(0.5, 0.5))
    model, oracle, cfg = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, num_layers=num_layers)
    ref = oracle(oracle_batch([s], [13, 29], 4.0, torch.float64), compute_stress=False)
    dev = torch.device("cuda:0")
    data = FakeLammpsData(s, 4.0, [13, 29], dev)
    assert data.ntotal > data.nlocal
    calc = TACELammpsCalc(model)
    assert calc.element_types == ["Al", "Cu"] and abs(calc.rcutfac - 2.0) < 1e-12
    calc.compute_forces(data)
    n = data.nlocal
    assert abs(data.energy - ref["energy"].item()) < 1e-8 * n
    assert (data.eatoms.cpu() - ref["node_energy"]).abs().max().item() < 1e-8
    # forces as LAMMPS assembles them from pair forces (newton on): f_i -= f_ij, f_j += f_ij, ghosts folded back
    f = torch.zeros(data.ntotal, 3, dtype=torch.float64, device=dev)
    f.index_add_(0, data.pair_i.long(), -data.pair_forces)
    f.index_add_(0, data.pair_j.long(), data.pair_forces)
    f[:n].index_add_(0, data.owner, f[n:])
    assert (f[:n].cpu() - ref["forces"]).abs().max().item() < 1e-7
    assert data.exchanges == 2 * (num_layers - 1)


def test_lammps_requires_kokkos_exchange():
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=4)
    model, _, _ = make_models(2, 32, [29], 4.0, 20.0, torch.float64)
    data = FakeLammpsData(s, 4.0, [29], torch.device("cuda:0"))
    calc = TACELammpsCalc(model)

    class NoExchange:
        nlocal, ntotal, npairs, elems = data.nlocal, data.ntotal, data.npairs, data.elems
    with pytest.raises(RuntimeError, match="KOKKOS"):
        calc.compute_forces(NoExchange())


class FakeSimState:
    """The attributes of a torch_sim SimState that the model interface reads."""

    def __init__(self, structures, device):
        b = synth.collate(structures)
        self.positions = torch.as_tensor(b["positions"], device=device)
        self.row_vector_cell = torch.as_tensor(b["lattice"], device=device)
        self.pbc = torch.tensor([True, True, True], device=device)
        self.atomic_numbers = torch.as_tensor(b["atomic_numbers"], device=device)
        self.system_idx = torch.as_tensor(b["batch"], device=device)


def test_torchsim_model_matches_oracle_and_reuses_cached_setup():
    from tace_b200.interface import TACETorchSimCalc

    structs = synth.random_crystals(3, seed=12, nmin=4, nmax=10, zmax=3)
    model, oracle, cfg = make_models(2, 32, [1, 2, 3], 4.5, 20.0, torch.float64)
    ref = oracle(oracle_batch(structs, [1, 2, 3], 4.5, torch.float64))
    dev = torch.device("cuda:0")
    calc = TACETorchSimCalc(model, device=dev, dtype=torch.float64)
    state = FakeSimState(structs, dev)
    for _ in range(2):  # the second call reuses the cached species / pointers
        out = calc(state)
        n_per = torch.tensor([len(s["positions"]) for s in structs], dtype=torch.float64)
        assert ((out["energy"].cpu() - ref["energy"]).abs() / n_per).max() < 1e-8
        assert (out["forces"].cpu() - ref["forces"]).abs().max() < 1e-7
        assert (out["stress"].cpu() - ref["stress"]).abs().max() < 1e-7
    assert calc.compute_forces and calc.compute_stress and calc.device == dev and calc.dtype == torch.float64
    with pytest.raises(NotImplementedError):
        TACETorchSimCalc(model, device=dev, enable_cue=True)
    # an element outside the model's table is refused
    state.atomic_numbers = state.atomic_numbers.clone()
    state.atomic_numbers[0] = 7
    with pytest.raises(ValueError):
        calc(state)


def test_lammps_mliap_with_the_tece_edge_block():
    """Edge-vector mode with ghost atoms for a model whose second interaction is the TECE edge block: ghost features arrive
    through the forward exchange, the gradients of ghost sources go back through the reverse exchange, and the gradient
    through the edge frames is part of the pair forces."""
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=6, species=(13, 29), fractions=(0.5, 0.5))
    model, oracle, cfg = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, radial={"apply_cutoff": False},
                                     tece={"num_head": 4, "edge_ace_hidden": 8, "mmax": 2})
    ref = oracle(oracle_batch([s], [13, 29], 4.0, torch.float64), compute_stress=False)
    dev = torch.device("cuda:0")
    data = FakeLammpsData(s, 4.0, [13, 29], dev)
    calc = TACELammpsCalc(model)
    calc.compute_forces(data)
    n = data.nlocal
    assert abs(data.energy - ref["energy"].item()) < 1e-8 * n
    f = torch.zeros(data.ntotal, 3, dtype=torch.float64, device=dev)
    f.index_add_(0, data.pair_i.long(), -data.pair_forces)
    f.index_add_(0, data.pair_j.long(), data.pair_forces)
    f[:n].index_add_(0, data.owner, f[n:])
    assert (f[:n].cpu() - ref["forces"]).abs().max().item() < 1e-7


@pytest.mark.parametrize("kw", [
    dict(zbl={"enable": True, "covalent_radii": {13: 1.5, 29: 1.6}}, scatter_norm="density"),
    dict(edge_update="element2", radial={"apply_cutoff": False, "bias": True, "hidden": [64, 64]}, gate_m0=False, use_alllayer=True),
    dict(product_nonlinear="silu_bilineargate", product_agnostic=True, resnet_linear_type="identity", correlation=2),
])
def test_lammps_mliap_with_model_options(kw):
    """Edge-vector mode with ghost atoms for the model options beyond the default: pair repulsion and learned edge density
    (sums over the edges into local atoms, species of ghost sources), element-dependent edge update with LayerNorm, gated
    bilinear product with identity skip."""
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=10, species=(13, 29), fractions=(0.5, 0.5))
    model, oracle, cfg = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, **kw)
    ref = oracle(oracle_batch([s], [13, 29], 4.0, torch.float64), compute_stress=False)
    dev = torch.device("cuda:0")
    data = FakeLammpsData(s, 4.0, [13, 29], dev)
    calc = TACELammpsCalc(model)
    calc.compute_forces(data)
    n = data.nlocal
    assert abs(data.energy - ref["energy"].item()) < 1e-8 * n
    assert (data.eatoms.cpu() - ref["node_energy"]).abs().max().item() < 1e-8
    f = torch.zeros(data.ntotal, 3, dtype=torch.float64, device=dev)
    f.index_add_(0, data.pair_i.long(), -data.pair_forces)
    f.index_add_(0, data.pair_j.long(), data.pair_forces)
    f[:n].index_add_(0, data.owner, f[n:])
    assert (f[:n].cpu() - ref["forces"]).abs().max().item() < 1e-7
