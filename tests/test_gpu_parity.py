"""CUDA path (through the C ABI) against the CPU oracle on identical seeded inputs and weights.

Tolerances are the ones the task states, absolute (``helpers.check_parity``): fp64 energy 1e-8 eV/atom and forces
1e-7 eV/A; fp32 energy 1e-5 eV/atom and forces 1e-4 eV/A (max-abs).  Stress is checked at the force tolerance, virials
(extensive) at the force tolerance times their largest entry.
"""
import numpy as np
import pytest
import torch

from tace_b200 import synth
from helpers import check_parity, make_models, oracle_batch, to_device

pytestmark = pytest.mark.gpu

TOL = {torch.float64: (1e-8, 1e-7), torch.float32: (1e-5, 1e-4)}


def run_case(structures, L, C, elements, cutoff, dtype, fidelity_idx=None, **kw):
    model, oracle, cfg = make_models(L, C, elements, cutoff, 20.0, dtype, **kw)
    data = oracle_batch(structures, elements, cutoff, dtype)
    if fidelity_idx is not None:
        data["fidelity_idx"] = torch.tensor(fidelity_idx, dtype=torch.int64)
    ref = oracle(data)
    out = model(to_device(data, torch.device("cuda:0")))
    torch.cuda.synchronize()
    check_parity(out, ref, data["ptr"], dtype, f"L{L} C{C}")
    return out, ref


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("L", [1, 2, 3])
def test_small_fcc(dtype, L):
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0)
    run_case([s], L, 32, [29], 4.0, dtype)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_triclinic_multi_element_batch(dtype):
    structs = synth.random_crystals(3, seed=5, nmin=4, nmax=12, zmax=3)
    run_case(structs, 3, 32, [1, 2, 3], 4.5, dtype)


def test_config1_cu256_fp64():
    """The fp64 reference-runnable configuration: FCC Cu 4x4x4, L=2, 64 channels, r_cut 5.0, fp64."""
    s = synth.workload_structures("cu256_fp64")[0]
    run_case([s], 2, 64, [29], 5.0, torch.float64)


def test_single_layer_and_correlation_one():
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=2, species=(13, 29), fractions=(0.5, 0.5))
    run_case([s], 2, 32, [13, 29], 4.0, torch.float64, num_layers=1)
    run_case([s], 2, 32, [13, 29], 4.0, torch.float64, correlation=1)


def test_three_layers():
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=3)
    run_case([s], 2, 32, [29], 4.0, torch.float64, num_layers=3)


def test_isolated_atom_and_empty_graph_edges():
    """A single atom in a big box has no edges: its read-out is masked (tace/models/blocks.py:347-369)."""
    lone = synth.Structure(positions=np.zeros((1, 3)), atomic_numbers=np.array([29]), cell=np.eye(3) * 30.0,
                           pbc=(True, True, True))
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0)
    out, ref = run_case([lone, s], 2, 32, [29], 4.0, torch.float64)
    assert out["forces"][0].abs().max().item() == 0.0


def test_isolated_atom_with_the_tece_edge_block():
    """The same batch through a model with the TECE edge block, and a batch that holds nothing but the lone atom (no edge
    at all: every per-edge stage has nothing to launch)."""
    lone = synth.Structure(positions=np.zeros((1, 3)), atomic_numbers=np.array([29]), cell=np.eye(3) * 30.0,
                           pbc=(True, True, True))
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0)
    kw = dict(radial={"apply_cutoff": False}, tece={"num_head": 4, "edge_ace_hidden": 8, "mmax": 2})
    out, ref = run_case([lone, s], 2, 32, [29], 4.0, torch.float64, **kw)
    assert out["forces"][0].abs().max().item() == 0.0
    out, ref = run_case([lone], 2, 32, [29], 4.0, torch.float64, **kw)
    assert out["forces"].abs().max().item() == 0.0


def test_input_not_mutated_and_repeatable():
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0)
    model, oracle, cfg = make_models(2, 32, [29], 4.0, 20.0, torch.float32)
    data = to_device(oracle_batch([s], [29], 4.0, torch.float32), torch.device("cuda:0"))
    before = {k: v.clone() for k, v in data.items()}
    a = model(data)
    b = model(data)
    for k in before:
        assert torch.equal(before[k], data[k]) and not data[k].requires_grad
    for k in ("energy", "forces", "stress"):
        assert torch.equal(a[k], b[k]), f"{k} differs between two identical calls"


def test_edge_vector_mode_matches_graph_mode():
    """LAMMPS-style input (edge vectors given) returns +dE/d(edge_vector)."""
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0)
    model, oracle, cfg = make_models(2, 32, [29], 4.0, 20.0, torch.float64, targets=("energy", "forces", "edge_forces"))
    data = oracle_batch([s], [29], 4.0, torch.float64)
    ref = oracle(data, compute_stress=False, compute_edge_forces=True)
    out = model(to_device(data, torch.device("cuda:0")))
    assert (out["edge_forces"].cpu() - ref["edge_forces"]).abs().max().item() < 1e-7
    assert (out["forces"].cpu() - ref["forces"]).abs().max().item() < 1e-7


@pytest.mark.parametrize("case", ["case_fcc32_L2_C32.npz", "case_bcc16_tece_L2_C32.npz"])
def test_golden_model_case(case):
    """The committed golden vectors (tests/golden/): the cgtp model and the one with the TECE edge block, fp64 and fp32."""
    import tace_b200
    from golden_util import load_case
    blob, sd, cfg, s = load_case(case)
    elements = [int(z) for z in blob["elements"]] if "elements" in blob else [29]
    for dtype in (torch.float64, torch.float32):
        prev = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            model = tace_b200.TensorModel(tace_b200.e3nnTACE(**cfg))
        finally:
            torch.set_default_dtype(prev)
        own = model.state_dict()
        model.load_state_dict({k: sd[k].to(own[k].dtype) for k in own})
        data = to_device(oracle_batch([s], elements, float(blob["cutoff"]), dtype), torch.device("cuda:0"))
        out = model(data)
        etol, ftol = TOL[dtype]
        n = len(s["positions"])
        assert abs(out["energy"].item() - blob["energy"].item()) / n <= etol
        assert np.abs(out["forces"].cpu().numpy() - blob["forces"]).max() <= ftol
        assert np.abs(out["stress"].cpu().numpy() - blob["stress"]).max() <= ftol


def test_full_size_properties_config2():
    """The headline configuration at full size (64 crystals, L=3, 128 channels, 89 elements, fp32): properties that need
    no oracle - net force per crystal ~ 0, run-to-run bit reproducibility, energy unchanged by a rigid shift
    and by relabelling atoms inside the batch order of the edge list."""
    from tace_b200.graph import build_batch
    wl = synth.WORKLOADS["crystals64_fp32"]
    structs = synth.workload_structures("crystals64_fp32")
    cfg = synth.model_config(wl["L"], wl["channels"], wl["cutoff"], wl["elements"], wl["avg_num_neighbors"])
    import tace_b200
    torch.manual_seed(0)
    model = tace_b200.TensorModel(tace_b200.e3nnTACE(**cfg))
    dev = torch.device("cuda:0")
    data = build_batch(synth.collate(structs), wl["elements"], wl["cutoff"], torch.float32, dev)
    a = model(data)
    b = model(data)
    assert model.device_error() == 0
    assert torch.equal(a["energy"], b["energy"]) and torch.equal(a["forces"], b["forces"])
    fscale = a["forces"].abs().max().item()
    net = torch.zeros(len(structs), 3, device=dev).index_add_(0, data["batch"], a["forces"])
    assert net.abs().max().item() <= 2e-4 * max(1.0, fscale)
    perm = torch.randperm(data["edge_index"].shape[1], device=dev)
    shuffled = dict(data, edge_index=data["edge_index"][:, perm].contiguous(), edge_shifts=data["edge_shifts"][perm].contiguous())
    c = model(shuffled)
    n_per = (data["ptr"][1:] - data["ptr"][:-1]).float()
    assert ((c["energy"] - a["energy"]).abs() / n_per).max().item() <= 1e-5
    assert (c["forces"] - a["forces"]).abs().max().item() <= 1e-4


def test_energy_of_large_graphs_is_the_sum_of_their_node_energies():
    """Graphs that average more than 16 384 atoms are summed in slices by several thread blocks and a second launch; two such graphs
    in one batch, each checked against the sum of its own node energies (fp64, a small model)."""
    from tace_b200.graph import build_batch
    structs = [synth.fcc_supercell(17, 3.61, 0.05, seed=31, species=(13, 29), fractions=(0.5, 0.5)),
               synth.fcc_supercell(16, 3.65, 0.05, seed=32, species=(13, 29), fractions=(0.2, 0.8))]
    model, _, _ = make_models(1, 32, [13, 29], 3.0, 12.0, torch.float64, num_layers=1, targets=("energy",))
    dev = torch.device("cuda:0")
    data = build_batch(synth.collate(structs), [13, 29], 3.0, torch.float64, dev)
    ptr = data["ptr"].tolist()
    assert (ptr[2] // 2) // 8192 >= 2  # two slices per graph at least
    out = model(data)
    assert model.device_error() == 0
    for g in range(2):
        total = out["node_energy"][ptr[g]:ptr[g + 1]].sum().item()
        assert abs(out["energy"][g].item() - total) <= 1e-9 * max(1.0, abs(total))


@pytest.mark.parametrize("L,C", [(2, 64), (3, 128)])
def test_fp32_tensor_core_channel_widths(L, C):
    """Channel counts for which fp32 models run the radial GEMMs and the per-rank linears on tcgen05."""
    structs = synth.random_crystals(2, seed=9, nmin=6, nmax=12, zmax=2)
    model_out, ref = run_case(structs, L, C, [1, 2], 4.5, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_graph_replay_is_bit_identical_and_follows_new_inputs(dtype):
    """From the third evaluation of one batch shape on, the pass is replayed as a CUDA graph: results must
    equal the launch-by-launch pass bit for bit, also when the caller's tensors live at new addresses and
    hold new coordinates."""
    structs = synth.random_crystals(3, seed=8, nmin=4, nmax=10, zmax=3)
    model, oracle, cfg = make_models(2, 32, [1, 2, 3], 4.5, 20.0, dtype)
    dev = torch.device("cuda:0")
    data = to_device(oracle_batch(structs, [1, 2, 3], 4.5, dtype), dev)
    first = {k: v.clone() for k, v in model(data).items() if v is not None}
    assert model.graph_replays() == 0
    keep = []
    for _ in range(3):
        again = {k: v.clone() for k, v in data.items()}  # fresh addresses
        keep.append(again)
        out = model(again)
        for k, v in first.items():
            assert torch.equal(out[k], v), k
    assert model.graph_replays() >= 2
    # same shapes, scaled coordinates: the replay must read the new values
    scaled = {k: v.clone() for k, v in data.items()}
    scaled["positions"] = data["positions"] * 1.01
    scaled["lattice"] = data["lattice"] * 1.01
    replayed = {k: v.clone() for k, v in model(scaled).items() if v is not None}
    model.set_graph_mode(False)
    direct = model(scaled)
    for k, v in replayed.items():
        assert torch.equal(direct[k], v), k
    assert not torch.equal(replayed["energy"], first["energy"])
    assert model.device_error() == 0


@pytest.mark.parametrize("dtype,num_layers,kw", [
    (torch.float64, 2, {}), (torch.float64, 3, {}), (torch.float32, 2, {}),
    (torch.float64, 2, dict(zbl={"enable": True, "covalent_radii": {13: 1.5, 29: 1.6}}, scatter_norm="density", num_fidelities=2)),
    (torch.float64, 3, dict(product_nonlinear="silu_bilineargate", resnet_linear_type="identity", edge_update="element2")),
])
def test_edge_chunked_pass_matches_the_whole_pass(dtype, num_layers, kw):
    """Chunks of target atoms with recomputed per-edge tensors (the mode used when a system's per-edge tensors
    do not fit) must give the whole-batch results up to the order of the per-source sums."""
    structs = [synth.fcc_supercell(4, 3.61, 0.05, seed=2, species=(13, 29), fractions=(0.4, 0.6)),
               synth.fcc_supercell(3, 3.61, 0.05, seed=3, species=(13, 29), fractions=(0.5, 0.5))]
    model, oracle, cfg = make_models(2, 32, [13, 29], 5.0, 40.0, dtype, num_layers=num_layers, **kw)
    dev = torch.device("cuda:0")
    data = to_device(oracle_batch(structs, [13, 29], 5.0, dtype), dev)
    if kw.get("num_fidelities"):
        data["fidelity_idx"] = torch.tensor([1, 0], device=dev)
    n_edges = data["edge_index"].shape[1]
    whole = {k: v.clone() for k, v in model(data).items() if v is not None}
    model.set_chunk_edges(2048)
    assert n_edges > 4 * 2048
    for _ in range(2):  # chunked passes are never replayed as graphs; the second call must agree too
        out = model(data)
        tol = 1e-11 if dtype == torch.float64 else 2e-5
        for k, v in whole.items():
            scale = max(1.0, v.abs().max().item())
            assert (out[k] - v).abs().max().item() <= tol * scale, k
    assert model.graph_replays() == 0
    assert model.device_error() == 0


def test_forces_and_stress_match_finite_differences_of_the_energy():
    """Central differences of the CUDA energy itself (fp64): F = -dE/dr, stress = (1/V) dE/d(strain) with the
    symmetric strain applied to positions and cell (tace/models/utils.py:50-79, adapter.py:106-116)."""
    s = synth.random_crystals(1, seed=21, nmin=6, nmax=6, zmax=3)[0]
    model, _, _ = make_models(2, 32, [1, 2, 3], 4.5, 20.0, torch.float64)
    dev = torch.device("cuda:0")

    def energy_of(struct):
        return model(to_device(oracle_batch([struct], [1, 2, 3], 4.5, torch.float64), dev))["energy"].item()

    base = model(to_device(oracle_batch([s], [1, 2, 3], 4.5, torch.float64), dev))
    forces, stress = base["forces"].cpu().numpy(), base["stress"].cpu().numpy()[0]
    h = 1e-5
    for i, k in [(0, 0), (3, 1), (5, 2)]:
        e = []
        for sign in (+1, -1):
            p = dict(s)
            p["positions"] = s["positions"].copy()
            p["positions"][i, k] += sign * h
            e.append(energy_of(p))
        assert abs(-(e[0] - e[1]) / (2 * h) - forces[i, k]) < 1e-6
    vol = abs(np.linalg.det(s["cell"]))
    for a, b in [(0, 0), (1, 2), (2, 0)]:
        e = []
        for sign in (+1, -1):
            eps = np.zeros((3, 3))
            eps[a, b] += 0.5 * sign * h
            eps[b, a] += 0.5 * sign * h
            p = dict(s)
            p["positions"] = s["positions"] @ (np.eye(3) + eps)
            p["cell"] = s["cell"] @ (np.eye(3) + eps)
            e.append(energy_of(p))
        fd = (e[0] - e[1]) / (2 * h) / vol
        assert abs(fd - stress[a, b]) < 1e-6, (a, b, fd, stress[a, b])
        assert abs(stress[a, b] - stress[b, a]) < 1e-12


@pytest.mark.parametrize("Lmax,lmax,num_layers,dtype", [(2, 3, 2, torch.float64), (1, 3, 3, torch.float64), (1, 2, 2, torch.float64),
                                                         (2, 3, 2, torch.float32)])
def test_node_rank_below_edge_rank(Lmax, lmax, num_layers, dtype):
    """Lmax < lmax (the reference's default is Lmax = 2, lmax = 3): node features between layers stop at Lmax while
    the angular features and the atomic basis go to lmax."""
    structs = synth.random_crystals(2, seed=31, nmin=4, nmax=9, zmax=3)
    run_case(structs, lmax, 32, [1, 2, 3], 4.5, dtype, Lmax=Lmax, num_layers=num_layers)


def test_reference_default_model_shape():
    """`e3nnTACE` with the reference defaults (Lmax 2, lmax 3, 64 channels, 2 layers, correlation 2)."""
    structs = synth.random_crystals(2, seed=32, nmin=4, nmax=8, zmax=2)
    run_case(structs, 3, 64, [1, 2], 5.0, torch.float32, Lmax=2)


@pytest.mark.parametrize("num_layers,Lmax,dtype", [(2, None, torch.float64), (3, 1, torch.float64), (2, None, torch.float32)])
def test_read_out_on_every_layer(num_layers, Lmax, dtype):
    """readout_emlp.use_alllayer: layers below the last add a linear read-out of their scalar channels."""
    structs = synth.random_crystals(2, seed=41, nmin=4, nmax=9, zmax=3)
    run_case(structs, 2, 32, [1, 2, 3], 4.5, dtype, num_layers=num_layers, Lmax=Lmax, use_alllayer=True)


@pytest.mark.parametrize("L,Lmax,dtype", [(2, None, torch.float64), (3, 2, torch.float64), (3, None, torch.float32)])
def test_scalars_through_silu_instead_of_a_gate(L, Lmax, dtype):
    """atomic_basis.gate_m0 = False: the e3nn Gate (scalars through SiLU, only ranks >= 1 gated)."""
    structs = synth.random_crystals(2, seed=43, nmin=4, nmax=9, zmax=3)
    run_case(structs, L, 32, [1, 2, 3], 4.5, dtype, Lmax=Lmax, gate_m0=False)


@pytest.mark.parametrize("L,Lmax,num_layers,dtype", [(2, None, 2, torch.float64), (3, 2, 2, torch.float64), (1, None, 3, torch.float64),
                                                      (3, None, 2, torch.float32)])
def test_correlation_three(L, Lmax, num_layers, dtype):
    """product_basis.correlation = 3: B = W1 A + W2 (A x A) + W3 ((A x A) x A)."""
    structs = synth.random_crystals(2, seed=47, nmin=4, nmax=8, zmax=3)
    run_case(structs, L, 32, [1, 2, 3], 4.5, dtype, Lmax=Lmax, num_layers=num_layers, correlation=3)


RADIAL_CASES = [
    ({"hidden": [64, 64]}, "identity"),
    ({"hidden": [64]}, "identity"),
    ({"bias": True}, "identity"),
    ({"apply_cutoff": False}, "identity"),
    ({"apply_cutoff": False, "bias": True, "hidden": [64, 64]}, "element2"),   # the radial section of example/train/tace.yaml
    ({}, "element2"),
]


@pytest.mark.parametrize("radial,edge_update", RADIAL_CASES)
def test_radial_mlp_options_and_element_dependent_edge_update(radial, edge_update):
    structs = synth.random_crystals(2, seed=53, nmin=4, nmax=9, zmax=3)
    run_case(structs, 2, 32, [1, 2, 3], 4.5, torch.float64, radial=radial, edge_update=edge_update)


def test_example_yaml_like_model_fp32_chunked_and_whole():
    """Lmax 2 / lmax 3, three layers, envelope after a biased two-layer radial MLP, element2 edge update, e3nn gate:
    the model section of the reference's example/train/tace.yaml except for its 48 channels."""
    structs = synth.random_crystals(2, seed=54, nmin=5, nmax=9, zmax=3)
    kw = dict(Lmax=2, num_layers=3, gate_m0=False, radial={"apply_cutoff": False, "bias": True, "hidden": [64, 64]},
              edge_update="element2")
    out, ref = run_case(structs, 3, 64, [1, 2, 3], 4.5, torch.float32, **kw)
    model, oracle, cfg = make_models(3, 64, [1, 2, 3], 4.5, 20.0, torch.float64, **kw)
    dev = torch.device("cuda:0")
    data = to_device(oracle_batch(structs, [1, 2, 3], 4.5, torch.float64), dev)
    whole = {k: v.clone() for k, v in model(data).items() if v is not None}
    model.set_chunk_edges(1024)
    chunked = model(data)
    for k, v in whole.items():
        assert (chunked[k] - v).abs().max().item() <= 1e-10 * max(1.0, v.abs().max().item()), k


@pytest.mark.parametrize("C,dtype", [(48, torch.float64), (48, torch.float32), (16, torch.float64)])
def test_channel_counts_that_are_not_multiples_of_32(C, dtype):
    """The reference's example configuration has 48 channels: such counts run zero-padded to the next multiple of 32."""
    structs = synth.random_crystals(2, seed=59, nmin=4, nmax=9, zmax=3)
    run_case(structs, 3, C, [1, 2, 3], 4.5, dtype, Lmax=2, gate_m0=False, edge_update="element2",
             radial={"apply_cutoff": False, "bias": True, "hidden": [64, 64]}, num_layers=3 if dtype == torch.float64 else 2)


@pytest.mark.parametrize("use_alllayer", [False, True])
def test_multi_fidelity_read_out(use_alllayer):
    """Three read-out heads (three `statistics` entries): every graph is evaluated with the head its `fidelity_idx`
    names; species scales and isolated-atom energies are per head.  Repeated calls (CUDA-graph replay) follow a
    changed `fidelity_idx`; without the key the head set by reset_fidelity_idx is used."""
    structs = synth.random_crystals(3, seed=21, nmin=4, nmax=10, zmax=3)
    dev = torch.device("cuda:0")
    model, oracle, _ = make_models(2, 32, [1, 2, 3], 4.5, 20.0, torch.float64, num_fidelities=3, use_alllayer=use_alllayer)
    data = oracle_batch(structs, [1, 2, 3], 4.5, torch.float64)
    seen = []
    for fid in ([2, 0, 1], [2, 0, 1], [1, 1, 0], [0, 2, 2]):
        data["fidelity_idx"] = torch.tensor(fid, dtype=torch.int64)
        ref = oracle(data)
        out = model(to_device(data, dev))
        assert (out["energy"].cpu() - ref["energy"]).abs().max().item() < 1e-8 * 10
        assert (out["node_energy"].cpu() - ref["node_energy"]).abs().max().item() < 1e-8
        assert (out["forces"].cpu() - ref["forces"]).abs().max().item() < 1e-7
        assert (out["stress"].cpu() - ref["stress"]).abs().max().item() < 1e-7
        seen.append(ref["energy"])
    assert model.graph_replays() >= 2
    assert (seen[0] - seen[2]).abs().max() > 1e-3  # the heads really differ
    del data["fidelity_idx"]
    model.reset_fidelity_idx(1)
    data1 = dict(data, fidelity_idx=torch.tensor([1, 1, 1]))
    out = model(to_device(data, dev))
    assert (out["energy"].cpu() - oracle(data1)["energy"]).abs().max().item() < 1e-7
    with pytest.raises(ValueError):
        model(to_device(dict(data, fidelity_idx=torch.tensor([0, 3, 1])), dev))
    assert model.device_error() == 0


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("scale_zbl", [True, False])
def test_zbl_pair_repulsion(dtype, scale_zbl):
    """short_range.zbl: screened nuclear repulsion inside the sum of the covalent radii, added to the read-out before
    (scale_zbl) or after the species scale; radii are given in the configuration (no ase here), chosen so that a good
    share of the pairs sits inside the envelope."""
    structs = synth.random_crystals(3, seed=23, nmin=4, nmax=10, zmax=3)
    zbl = {"enable": True, "covalent_radii": {1: 0.9, 2: 1.3, 3: 1.6}}
    out, ref = run_case(structs, 2, 32, [1, 2, 3], 4.5, dtype, zbl=zbl, scale_zbl=scale_zbl)
    base, _ = run_case(structs, 2, 32, [1, 2, 3], 4.5, dtype)
    assert (out["energy"] - base["energy"]).abs().max().item() > 1e-2  # the term is really there


@pytest.mark.parametrize("scatter_norm,radial", [
    ("density", {}), ("density", {"apply_cutoff": False, "bias": True}), ("no_cutoff_density", {"apply_cutoff": False}),
])
def test_learned_edge_density_normalisation(scatter_norm, radial):
    """atomic_basis.scatter_norm = density / no_cutoff_density: messages divided by alpha + beta * sum over the incoming
    edges of tanh(MLP(radial)^2), with the envelope factor where the reference applies it."""
    structs = synth.random_crystals(3, seed=27, nmin=4, nmax=10, zmax=3)
    for dtype in (torch.float64, torch.float32):
        run_case(structs, 2, 32, [1, 2, 3], 4.5, dtype, scatter_norm=scatter_norm, radial=radial)


@pytest.mark.parametrize("resnet_linear_type,product_agnostic", [("identity", False), ("agnostic", True), ("identity", True)])
def test_skip_connection_types_and_species_agnostic_product(resnet_linear_type, product_agnostic):
    """resnet.linear_type = identity (ranks copied over, none for the last layer but the scalars) / agnostic (one linear for
    every species) and product_basis.agnostic (one coefficient matrix for every species); three layers so that a middle
    layer (equal ranks in and out) and the last layer (scalars only) are both covered, node rank below edge rank."""
    structs = synth.random_crystals(3, seed=29, nmin=4, nmax=10, zmax=3)
    for dtype in (torch.float64, torch.float32):
        run_case(structs, 3, 32, [1, 2, 3], 4.5, dtype, num_layers=3, Lmax=2, resnet_linear_type=resnet_linear_type,
                 product_agnostic=product_agnostic)


@pytest.mark.parametrize("L,Lmax,num_layers", [(2, None, 2), (3, 2, 3)])
def test_gated_bilinear_product(L, Lmax, num_layers):
    """product_basis.nonlinear = silu_bilineargate: the product's own linear_up makes two factors and one SiLU gate per
    (path, channel); second-order basis = gate * (x (x) [y, 1]), first-order coefficients on x."""
    structs = synth.random_crystals(3, seed=31, nmin=4, nmax=10, zmax=3)
    for dtype in (torch.float64, torch.float32):
        run_case(structs, L, 32, [1, 2, 3], 4.5, dtype, Lmax=Lmax, num_layers=num_layers, product_nonlinear="silu_bilineargate")
    run_case(structs, 2, 64, [1, 2, 3], 4.5, torch.float32, product_nonlinear="silu_bilineargate", product_agnostic=True,
             resnet_linear_type="identity")


@pytest.mark.parametrize("L,mmax,gate_m0,radial,num_layers", [
    (2, 2, True, {"apply_cutoff": False}, 2),
    (3, 2, False, {"apply_cutoff": False, "bias": True, "hidden": [64, 64]}, 2),
    (2, 1, True, {}, 3),
])
def test_tece_edge_block(L, mmax, gate_m0, radial, num_layers):
    """atomic_basis.type = [cgtp, uv_so2, ...]: edge-frame rotation with recursive Wigner matrices, SO(2) linears, gate, edge
    cluster expansion, rotary attention normalised over the incoming edges; gradients through the frames in forward mode."""
    structs = synth.random_crystals(2, seed=33, nmin=4, nmax=8, zmax=3)
    tece = {"num_head": 4, "edge_ace_hidden": 8, "mmax": mmax}
    for dtype in (torch.float64, torch.float32):
        run_case(structs, L, 32, [1, 2, 3], 4.0, dtype, gate_m0=gate_m0, radial=radial, num_layers=num_layers, tece=tece)


def test_tece_example_configuration_small():
    """The model of benchmark configuration 4 (the reference's example TECE file: cgtp then uv_so2, element-dependent edge
    update with LayerNorm, envelope after a biased two-layer radial MLP, e3nn gate, identity skip, species-agnostic gated
    bilinear product) at 32 channels on a small five-component BCC cell, fp64 and fp32; repeated calls replay a CUDA graph."""
    s = synth.bcc_supercell(2, 2.87, 0.08, seed=3, species=(23, 24, 26, 27, 28))
    kw = dict(synth.WORKLOADS["tece8192_fp32"]["model"])
    kw["tece"] = {"num_head": 4, "edge_ace_hidden": 8, "mmax": 2}
    for dtype in (torch.float64, torch.float32):
        run_case([s], 3, 32, [23, 24, 26, 27, 28], 4.0, dtype, **kw)
    model, oracle, _ = make_models(3, 32, [23, 24, 26, 27, 28], 4.0, 20.0, torch.float64, **kw)
    data = oracle_batch([s], [23, 24, 26, 27, 28], 4.0, torch.float64)
    dev_data = to_device(data, torch.device("cuda:0"))
    first = model(dev_data)
    for _ in range(3):
        again = model(dev_data)
    assert model.graph_replays() >= 2
    assert torch.equal(first["forces"], again["forces"]) and torch.equal(first["energy"], again["energy"])


def test_tece_edge_block_wide_head():
    """One head over 64 channels: wider than a warp, so the attention kernels take their per-(edge, head) form."""
    structs = synth.random_crystals(2, seed=35, nmin=4, nmax=8, zmax=3)
    run_case(structs, 2, 64, [1, 2, 3], 4.0, torch.float64, radial={"apply_cutoff": False}, tece={"num_head": 1, "edge_ace_hidden": 8, "mmax": 2})


def test_full_size_properties_config4():
    """Benchmark configuration 4 at full size (TECE model, 8 192 atoms, 526 k edges, L = 3, 128 channels, fp32): properties
    that need no oracle - net force ~ 0, run-to-run bit reproducibility (graph replay included), energy and forces unchanged
    by a rigid shift of all atoms and by a permutation of the edge list."""
    import tace_b200
    from tace_b200.graph import build_batch
    wl = synth.WORKLOADS["tece8192_fp32"]
    structs = synth.workload_structures("tece8192_fp32")
    cfg = synth.model_config(wl["L"], wl["channels"], wl["cutoff"], wl["elements"], wl["avg_num_neighbors"], **wl["model"])
    torch.manual_seed(0)
    model = tace_b200.TensorModel(tace_b200.e3nnTACE(**cfg))
    dev = torch.device("cuda:0")
    data = build_batch(synth.collate(structs), wl["elements"], wl["cutoff"], torch.float32, dev)
    a = model(data)
    b = model(data)
    c = model(data)
    assert model.device_error() == 0
    for other in (b, c):
        assert torch.equal(a["energy"], other["energy"]) and torch.equal(a["forces"], other["forces"])
    n = a["forces"].shape[0]
    fscale = a["forces"].abs().max().item()
    assert torch.isfinite(a["forces"]).all() and fscale > 0
    assert a["forces"].sum(0).abs().max().item() <= 1e-5 * n * max(1.0, fscale)
    shifted = dict(data, positions=data["positions"] + torch.tensor([0.31, -0.27, 0.19], device=dev, dtype=data["positions"].dtype))
    d = model(shifted)
    assert abs(d["energy"].item() - a["energy"].item()) / n <= 1e-5
    assert (d["forces"] - a["forces"]).abs().max().item() <= 1e-4
    perm = torch.randperm(data["edge_index"].shape[1], device=dev)
    shuffled = dict(data, edge_index=data["edge_index"][:, perm].contiguous(), edge_shifts=data["edge_shifts"][perm].contiguous())
    e = model(shuffled)
    assert abs(e["energy"].item() - a["energy"].item()) / n <= 1e-5
    assert (e["forces"] - a["forces"]).abs().max().item() <= 1e-4
    model.release()
    del model
    torch.cuda.empty_cache()


@pytest.mark.parametrize("L,C,radial", [(3, 64, {}), (2, 64, {"apply_cutoff": False, "bias": True, "hidden": [64, 64]}), (2, 32, {"hidden": [64]})])
def test_tabulated_radial_weights_match_the_per_edge_mlp(L, C, radial):
    """fp32 models with the identity edge update read the path weights from a table of the edge length (cubic Hermite)
    instead of running the radial MLP per edge.  Both routes must agree far inside the fp32 tolerances, whole and
    chunked, and both must match the oracle."""
    structs = [synth.fcc_supercell(3, 3.61, 0.05, seed=61, species=(1, 2, 3), fractions=(0.3, 0.3, 0.4)),
               synth.random_crystals(1, seed=61, nmin=10, nmax=14, zmax=3)[0]]
    model, oracle, cfg = make_models(L, C, [1, 2, 3], 5.0, 20.0, torch.float32, radial=radial)
    data = oracle_batch(structs, [1, 2, 3], 5.0, torch.float32)
    dev_data = to_device(data, torch.device("cuda:0"))
    ref = oracle(data)
    tab = {k: v.clone() for k, v in model(dev_data).items() if v is not None}
    assert model.uses_radial_table
    check_parity(tab, ref, data["ptr"], torch.float32, f"table L{L} C{C}")
    model.set_chunk_edges(1024)
    assert data["edge_index"].shape[1] > 2 * 1024
    chunked = {k: v.clone() for k, v in model(dev_data).items() if v is not None}
    model.set_chunk_edges(1 << 21)
    model.set_radial_table(False)
    mlp = model(dev_data)
    assert not model.uses_radial_table
    check_parity(mlp, ref, data["ptr"], torch.float32, f"per-edge MLP L{L} C{C}")
    n_per = (data["ptr"][1:] - data["ptr"][:-1]).float()
    for other, what in ((chunked, "chunked table"), (mlp, "per-edge MLP")):
        de = ((tab["energy"] - other["energy"]).abs().cpu() / n_per).max().item()
        df = (tab["forces"] - other["forces"]).abs().max().item()
        print(f"table vs {what}: dE/atom = {de:.3e}, dF = {df:.3e}")
        assert de <= 2e-6 and df <= 2e-5, what
    assert model.device_error() == 0
