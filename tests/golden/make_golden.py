#!/usr/bin/env python
"""Regenerates the golden fixtures in this directory:  python tests/golden/make_golden.py

The reference itself cannot be imported offline (it needs e3nn, ase, matscipy), and its own tests
hold no energy / force / neighbour-list value for this path, so these vectors are outputs of the
CPU oracle (``oracle/``), stored to pin it - and the CUDA path - against regressions.  The only
reference-held numbers are the three activation constants of ``tace/models/mlp.py:34,43,52``,
stored in ``o3_tables.npz`` next to the tables they are checked with.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

from helpers import make_models, oracle_batch  # noqa: E402
from oracle import o3  # noqa: E402
from oracle.neighbour_list import neighbour_list  # noqa: E402
from tace_b200 import synth  # noqa: E402


def store_case(name, structure, elements, cutoff, dtype_weights=np.float32, **model_kw):
    """One model case with its weights (rounded to fp32) and the oracle's fp64 outputs for those weights; the model
    configuration travels as JSON so that the loader needs no per-case code."""
    import json

    from oracle.model import build_oracle
    model, _, cfg = make_models(model_kw.pop("L"), model_kw.pop("C"), elements, cutoff, 20.0, torch.float64, seed=0, **model_kw)
    data = oracle_batch([structure], elements, cutoff, torch.float64)
    sd = {k: v.numpy().astype(dtype_weights if v.is_floating_point() else np.int64) for k, v in model.state_dict().items()}
    sd64 = {k: torch.from_numpy(v.astype(np.float64) if v.dtype == dtype_weights else v) for k, v in sd.items()}
    ref = build_oracle(cfg, sd64, torch.float64)(data)
    np.savez_compressed(os.path.join(HERE, name), positions=structure["positions"], cell=structure["cell"],
                        atomic_numbers=structure["atomic_numbers"], cutoff=cutoff, avg_num_neighbors=20.0,
                        elements=np.asarray(elements), cfg_json=np.array(json.dumps(cfg)),
                        energy=ref["energy"].numpy(), forces=ref["forces"].numpy(), stress=ref["stress"].numpy(),
                        node_energy=ref["node_energy"].numpy(), **{"sd:" + k: v for k, v in sd.items()})


def tece_case():
    # --- model case B: cgtp layer + TECE edge block (two species, BCC 2 x 2 x 2), weights stored
    s = synth.bcc_supercell(2, 2.87, 0.08, seed=3, species=(26, 28))
    store_case("case_bcc16_tece_L2_C32.npz", s, [26, 28], 4.0, L=2, C=32, radial={"apply_cutoff": False},
               tece={"num_head": 4, "edge_ace_hidden": 8, "mmax": 2})


def main():
    if "--tece-only" in sys.argv:
        tece_case()
        return
    # --- conventions: Wigner 3j, spherical harmonics, activation constants
    tables = {"activation_constants_reference": np.array([1.6791767923989418, 1.8467055342154763, 1.5937334472592695])}
    for l1 in range(4):
        for l2 in range(4):
            for l3 in range(abs(l1 - l2), min(3, l1 + l2) + 1):
                if (l1 + l2 + l3) % 2 == 0:
                    tables[f"w3j_{l1}{l2}{l3}"] = o3.wigner_3j(l1, l2, l3).numpy()
    pts = torch.tensor([[0.3, -0.5, 0.8], [1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [-0.2, 0.9, 0.4]], dtype=torch.float64)
    tables["sh_points"] = pts.numpy()
    tables["sh_values_component"] = o3.spherical_harmonics(3, pts, "component").numpy()
    np.savez(os.path.join(HERE, "o3_tables.npz"), **tables)

    # --- model case A: weights stored, so the fixture does not depend on torch's random stream
    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0)
    model, oracle, cfg = make_models(2, 32, [29], 4.0, 20.0, torch.float64, seed=0)
    data = oracle_batch([s], [29], 4.0, torch.float64)
    ref = oracle(data)
    sd = {k: v.numpy().astype(np.float32 if v.is_floating_point() else np.int64) for k, v in model.state_dict().items()}
    np.savez_compressed(os.path.join(HERE, "case_fcc32_L2_C32.npz"), positions=s["positions"], cell=s["cell"],
                        atomic_numbers=s["atomic_numbers"], cutoff=4.0, avg_num_neighbors=20.0,
                        edge_index=data["edge_index"].numpy(), edge_shifts=data["edge_shifts"].numpy(),
                        energy=ref["energy"].numpy(), forces=ref["forces"].numpy(), stress=ref["stress"].numpy(),
                        node_energy=ref["node_energy"].numpy(),
                        **{"sd:" + k: v for k, v in sd.items()})
    # NOTE: weights are stored in fp32; the stored outputs are those of the fp32-rounded weights
    sd64 = {k: torch.from_numpy(v.astype(np.float64) if v.dtype == np.float32 else v) for k, v in sd.items()}
    from oracle.model import build_oracle
    ref = build_oracle(cfg, sd64, torch.float64)(data)
    blob = dict(np.load(os.path.join(HERE, "case_fcc32_L2_C32.npz")))
    blob.update(energy=ref["energy"].numpy(), forces=ref["forces"].numpy(), stress=ref["stress"].numpy(),
                node_energy=ref["node_energy"].numpy())
    np.savez_compressed(os.path.join(HERE, "case_fcc32_L2_C32.npz"), **blob)

    # --- neighbour-list case: triclinic cell narrower than the cutoff (self images, several shells of images)
    t = synth.random_crystals(1, seed=7, nmin=5, nmax=5)[0]
    ei, es = neighbour_list(t["positions"], t["cell"], t["pbc"], 6.0)
    np.savez_compressed(os.path.join(HERE, "neighbour_list_triclinic5.npz"), positions=t["positions"], cell=t["cell"],
                        cutoff=6.0, edge_index=ei, edge_shifts=es)
    tece_case()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
