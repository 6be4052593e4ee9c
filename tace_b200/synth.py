"""Seeded synthetic structures and model configurations for tests and benchmarks.

The reference's published models are trained on public materials datasets that
are not needed here: every workload below is generated from a fixed seed with
the stated sizes, densities and value distributions.
"""

from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np


class Structure(dict):
    """positions float64[N,3], atomic_numbers int64[N], cell float64[3,3], pbc (3 bools)."""


def _structure(positions, numbers, cell, pbc=(True, True, True)) -> Structure:
    return Structure(
        positions=np.ascontiguousarray(positions, dtype=np.float64),
        atomic_numbers=np.ascontiguousarray(numbers, dtype=np.int64),
        cell=np.ascontiguousarray(cell, dtype=np.float64).reshape(3, 3),
        pbc=tuple(bool(p) for p in pbc),
    )


def fcc_supercell(reps: int, a: float, sigma: float, seed: int, species=(29,), fractions=(1.0,)) -> Structure:
    """FCC conventional cells repeated ``reps`` times per axis, Gaussian positional noise,
    species drawn independently per site with the given probabilities."""
    rng = np.random.default_rng(seed)
    basis = np.array([[0, 0, 0], [0, 0.5, 0.5], [0.5, 0, 0.5], [0.5, 0.5, 0]], dtype=np.float64)
    grid = np.stack(np.meshgrid(*[np.arange(reps)] * 3, indexing="ij"), axis=-1).reshape(-1, 1, 3)
    pos = ((grid + basis[None]).reshape(-1, 3)) * a
    pos = pos + rng.normal(0.0, sigma, size=pos.shape)
    if len(species) == 1:
        z = np.full(pos.shape[0], species[0], dtype=np.int64)
    else:
        z = rng.choice(np.asarray(species, dtype=np.int64), size=pos.shape[0], p=np.asarray(fractions))
    return _structure(pos, z, np.eye(3) * reps * a)


def bcc_supercell(reps: int, a: float, sigma: float, seed: int, species: Sequence[int]) -> Structure:
    """BCC cells with an equimolar random permutation of ``species`` and Gaussian noise."""
    rng = np.random.default_rng(seed)
    basis = np.array([[0, 0, 0], [0.5, 0.5, 0.5]], dtype=np.float64)
    grid = np.stack(np.meshgrid(*[np.arange(reps)] * 3, indexing="ij"), axis=-1).reshape(-1, 1, 3)
    pos = ((grid + basis[None]).reshape(-1, 3)) * a
    n = pos.shape[0]
    z = np.resize(np.asarray(species, dtype=np.int64), n)
    z = rng.permutation(z)
    pos = pos + rng.normal(0.0, sigma, size=pos.shape)
    return _structure(pos, z, np.eye(3) * reps * a)


def _cell_from_lengths_angles(lengths, angles_deg) -> np.ndarray:
    a, b, c = lengths
    al, be, ga = np.deg2rad(angles_deg)
    va = np.array([a, 0.0, 0.0])
    vb = np.array([b * np.cos(ga), b * np.sin(ga), 0.0])
    cx = c * np.cos(be)
    cy = c * (np.cos(al) - np.cos(be) * np.cos(ga)) / np.sin(ga)
    cz = np.sqrt(max(c * c - cx * cx - cy * cy, 1e-12))
    return np.stack([va, vb, np.array([cx, cy, cz])])


def random_crystals(num: int = 64, seed: int = 1, nmin: int = 8, nmax: int = 64, zmax: int = 89,
                    density: float = 0.07, min_dist: float = 1.0) -> List[Structure]:
    """Random triclinic crystals: atom count U{nmin..nmax}, species U{1..zmax}, lengths U[4,12] A,
    angles U[70,110] deg, cell rescaled to ``density`` atoms/A^3, uniform fractional coordinates
    with rejection of any pair (periodic copies included) closer than ``min_dist``."""
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(num):
        n = int(rng.integers(nmin, nmax + 1))
        z = rng.integers(1, zmax + 1, size=n)
        cell = _cell_from_lengths_angles(rng.uniform(4.0, 12.0, 3), rng.uniform(70.0, 110.0, 3))
        cell *= (n / density / abs(np.linalg.det(cell))) ** (1.0 / 3.0)
        images = np.stack(np.meshgrid(*[np.arange(-1, 2)] * 3, indexing="ij"), axis=-1).reshape(-1, 3)
        frac = np.zeros((0, 3))
        while frac.shape[0] < n:
            f = rng.uniform(0.0, 1.0, 3)
            cand = np.concatenate([frac, f[None]]) if frac.size else f[None]
            d = (cand[None, :, :] - f[None, None, :] + images[:, None, :]) @ cell  # [27, m, 3]
            dist = np.linalg.norm(d, axis=-1)
            dist[13, -1] = np.inf  # the candidate with itself at zero shift
            if dist.min() >= min_dist:
                frac = cand
        out.append(_structure(frac @ cell, z, cell))
    return out


def water_box(n_side: int = 23, box: float = 68.6, sigma: float = 0.03, seed: int = 2, n_mol: int = 10800) -> Structure:
    """Rigid H2O molecules (O-H 0.9572 A, H-O-H 104.52 deg) on a jittered grid with uniform random
    orientations and Gaussian noise.  Defaults give 32,400 atoms at 1.0 g/cm^3."""
    rng = np.random.default_rng(seed)
    assert n_side**3 >= n_mol
    sites = np.stack(np.meshgrid(*[np.arange(n_side)] * 3, indexing="ij"), axis=-1).reshape(-1, 3)
    sites = sites[rng.permutation(sites.shape[0])[:n_mol]]
    h = box / n_side
    centers = (sites + 0.5) * h + rng.uniform(-0.15, 0.15, size=(n_mol, 3)) * h
    half = np.deg2rad(104.52) / 2.0
    mol = np.array([[0.0, 0.0, 0.0],
                    [0.9572 * np.sin(half), 0.9572 * np.cos(half), 0.0],
                    [-0.9572 * np.sin(half), 0.9572 * np.cos(half), 0.0]])
    q = rng.normal(size=(n_mol, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    w, x, y, z = q.T
    rot = np.stack([
        np.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)], -1),
        np.stack([2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)], -1),
        np.stack([2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], -1),
    ], axis=1)
    pos = centers[:, None, :] + np.einsum("nij,aj->nai", rot, mol)
    pos = pos.reshape(-1, 3) + rng.normal(0.0, sigma, size=(3 * n_mol, 3))
    zs = np.tile(np.array([8, 1, 1], dtype=np.int64), n_mol)
    return _structure(pos, zs, np.eye(3) * box)


def collate(structures: Sequence[Structure]) -> Dict[str, np.ndarray]:
    """Concatenate structures into one batch: positions, atomic_numbers, lattice[B,3,3],
    pbc[B,3], batch[N], ptr[B+1] (the PyG batching the reference uses, tace/models/adapter.py:326-340)."""
    counts = [s["positions"].shape[0] for s in structures]
    ptr = np.zeros(len(structures) + 1, dtype=np.int64)
    ptr[1:] = np.cumsum(counts)
    return {
        "positions": np.concatenate([s["positions"] for s in structures]),
        "atomic_numbers": np.concatenate([s["atomic_numbers"] for s in structures]),
        "lattice": np.stack([s["cell"] for s in structures]),
        "pbc": np.array([s["pbc"] for s in structures], dtype=np.uint8),
        "batch": np.repeat(np.arange(len(structures), dtype=np.int64), counts),
        "ptr": ptr,
    }


def statistics(atomic_numbers: Sequence[int], avg_num_neighbors: float, num_fidelities: int = 1) -> List[Dict]:
    """The statistics list the model constructor consumes (tace/models/_e3nn/default.py:251-280), one entry per
    fidelity: zero isolated-atom energies, unit force scale."""
    zs = sorted(int(z) for z in set(atomic_numbers))
    return [{
        "atomic_numbers": zs,
        "avg_num_neighbors": float(avg_num_neighbors),
        "atomic_energy": {z: 0.0 for z in zs},
        "rms_forces": {z: 1.0 for z in zs},
    } for _ in range(num_fidelities)]


def model_config(L: int, channels: int, cutoff: float, elements: Sequence[int], avg_num_neighbors: float,
                 num_layers: int = 2, correlation: int = 2, target_property=("energy", "forces", "stress"),
                 Lmax: int = None, use_alllayer: bool = False, gate_m0: bool = True, radial: Dict = None,
                 edge_update: str = "identity", num_fidelities: int = 1, zbl: Dict = None, scale_zbl: bool = True,
                 scatter_norm: str = "avg_num_neighbors", resnet_linear_type: str = "aware",
                 product_agnostic: bool = False, product_nonlinear: str = None, tece: Dict = None) -> Dict:
    """Keyword arguments for ``tace_b200.models.e3nnTACE`` (cgtp interaction, cgtp product).  ``L`` is the edge
    rank ``lmax``; the node rank ``Lmax`` defaults to it."""
    atomic_basis = {"gate_m0": bool(gate_m0), "scatter_norm": scatter_norm}
    extra = {}
    if tece:  # every interaction above the first is the TECE edge block: {"num_head", "edge_ace_hidden", "mmax", "edge_nonlinear"}
        atomic_basis.update(type=["cgtp"] + ["uv_so2"] * (num_layers - 1), num_head=tece.get("num_head", 1),
                            edge_ace_hidden=tece.get("edge_ace_hidden"), edge_nonlinear=tece.get("edge_nonlinear", "so2_sigmoid_gate"))
        extra["mmax"] = tece.get("mmax", 2)
    return {
        **extra,
        "Lmax": L if Lmax is None else Lmax, "lmax": L, "num_layers": num_layers, "num_channel": channels, "cutoff": float(cutoff),
        "statistics": statistics(elements, avg_num_neighbors, num_fidelities),
        "target_property": list(target_property), "max_neighbors": None,
        "product_basis": {"correlation": correlation, "agnostic": bool(product_agnostic), "nonlinear": product_nonlinear},
        "resnet": {"linear_type": resnet_linear_type},
        "readout_emlp": {"use_alllayer": bool(use_alllayer)},
        "atomic_basis": atomic_basis,
        "radial_basis": dict(radial or {}),
        "edge_update": {"type": edge_update},
        "short_range": {"zbl": dict(zbl or {"enable": False})},
        "scale_shift": {"scale_zbl": bool(scale_zbl)},
    }


# The workloads named by the benchmark contract.  ``avg_num_neighbors`` is the measured mean degree of
# the generated input, frozen here so the model definition does not depend on the neighbour list.
WORKLOADS = {
    "cu256_fp64": dict(L=2, channels=64, cutoff=5.0, elements=[29], avg_num_neighbors=42.75, dtype="float64"),
    "crystals64_fp32": dict(L=3, channels=128, cutoff=6.0, elements=list(range(1, 90)), avg_num_neighbors=63.3,
                            dtype="float32"),
    # a quarter of the batch above, used for profiler captures
    "crystals16_fp32": dict(L=3, channels=128, cutoff=6.0, elements=list(range(1, 90)), avg_num_neighbors=63.3,
                            dtype="float32"),
    "water32400_fp32": dict(L=3, channels=128, cutoff=6.0, elements=[1, 8], avg_num_neighbors=90.0, dtype="float32",
                            cpu_sample="water192_fp32"),
    # 64 molecules at the same density, built by the same rules: the CPU baseline's sample of configuration 3
    "water192_fp32": dict(L=3, channels=128, cutoff=6.0, elements=[1, 8], avg_num_neighbors=90.0, dtype="float32"),
    "cual1m_fp32": dict(L=2, channels=64, cutoff=5.0, elements=[13, 29], avg_num_neighbors=42.1, dtype="float32"),
    # benchmark configuration 4: the TECE model of the reference's example/train/tece.yaml at L = 3, C = 128 on a five-component BCC alloy
    "tece8192_fp32": dict(L=3, channels=128, cutoff=6.0, elements=[23, 24, 26, 27, 28], avg_num_neighbors=64.0, dtype="float32",
                          cpu_sample="tece1024_fp32",
                          model=dict(gate_m0=False, edge_update="element2", radial={"apply_cutoff": False, "bias": True, "hidden": [64, 64]},
                                     resnet_linear_type="identity", product_agnostic=True, product_nonlinear="silu_bilineargate",
                                     tece={"num_head": 8, "edge_ace_hidden": 32, "mmax": 2})),
    # the same model on 8 x 8 x 8 cells (1 024 atoms, 65 770 edges, about 8 GB on the device): profiler captures, CPU baseline
    "tece1024_fp32": dict(L=3, channels=128, cutoff=6.0, elements=[23, 24, 26, 27, 28], avg_num_neighbors=64.0, dtype="float32",
                          model=dict(gate_m0=False, edge_update="element2", radial={"apply_cutoff": False, "bias": True, "hidden": [64, 64]},
                                     resnet_linear_type="identity", product_agnostic=True, product_nonlinear="silu_bilineargate",
                                     tece={"num_head": 8, "edge_ace_hidden": 32, "mmax": 2})),
    # the same model on 4 x 4 x 4 cells, for quick checks
    "tece128_fp32": dict(L=3, channels=128, cutoff=6.0, elements=[23, 24, 26, 27, 28], avg_num_neighbors=64.0, dtype="float32",
                         model=dict(gate_m0=False, edge_update="element2", radial={"apply_cutoff": False, "bias": True, "hidden": [64, 64]},
                                    resnet_linear_type="identity", product_agnostic=True, product_nonlinear="silu_bilineargate",
                                    tece={"num_head": 8, "edge_ace_hidden": 32, "mmax": 2})),
    # one eighth of the system above (the share of one GPU in an 8-GPU run), for development runs
    "cual131k_fp32": dict(L=2, channels=64, cutoff=5.0, elements=[13, 29], avg_num_neighbors=42.1, dtype="float32"),
}
MD_WORKLOADS = {"cual1m_fp32": 64, "cual131k_fp32": 32}  # FCC cells per side


def workload_structures(name: str) -> List[Structure]:
    if name == "cu256_fp64":
        return [fcc_supercell(4, 3.61, 0.05, seed=0)]
    if name == "crystals64_fp32":
        return random_crystals(64, seed=1)
    if name == "crystals16_fp32":
        return random_crystals(16, seed=1)
    if name == "water32400_fp32":
        return [water_box()]
    if name == "water192_fp32":
        return [water_box(n_side=4, box=68.6 * (64 / 10800) ** (1.0 / 3.0), n_mol=64)]
    if name == "tece8192_fp32":
        return [bcc_supercell(16, 2.87, 0.08, seed=3, species=(23, 24, 26, 27, 28))]
    if name == "tece1024_fp32":  # 8 x 8 x 8 cells: the CPU baseline's sample of configuration 4
        return [bcc_supercell(8, 2.87, 0.08, seed=3, species=(23, 24, 26, 27, 28))]
    if name == "tece128_fp32":
        return [bcc_supercell(4, 2.87, 0.08, seed=3, species=(23, 24, 26, 27, 28))]
    if name in MD_WORKLOADS:
        return [fcc_supercell(MD_WORKLOADS[name], 3.65, 0.05, seed=4, species=(13, 29), fractions=(0.1, 0.9))]
    raise KeyError(name)
