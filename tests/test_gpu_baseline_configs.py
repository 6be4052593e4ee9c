"""The benchmark configurations on their own models and inputs, CUDA path against the CPU oracle, with the task's
absolute tolerances (fp32: 1e-5 eV/atom, 1e-4 eV/A; fp64: 1e-8 eV/atom, 1e-7 eV/A), and the CUDA path against the
fixtures computed by the reference's own source files (``tests/golden/ref_*.npz``).

The oracle is a dense PyTorch model, so it sees each configuration at a size it finishes in seconds: the smallest
crystals of configuration 2's batch (the GPU evaluates the whole batch), a 64-molecule water box built by the rules of
configuration 3, configuration 4's full model on a 3 x 3 x 3 cell, configuration 5's model on a 4 x 4 x 4 cell through
the domain-decomposed MD driver.
"""
import json
import os

import numpy as np
import pytest
import torch

import tace_b200
from helpers import check_parity, make_models, oracle_batch, to_device
from tace_b200 import synth

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _subset(out, data, graphs):
    """The rows of a batched result that belong to ``graphs``, renumbered as a batch of their own."""
    ptr = data["ptr"].cpu()
    rows = torch.cat([torch.arange(int(ptr[g]), int(ptr[g + 1])) for g in graphs])
    g = torch.tensor(graphs)
    sub = {"energy": out["energy"].cpu()[g], "forces": out["forces"].cpu()[rows], "node_energy": out["node_energy"].cpu()[rows]}
    if out.get("stress") is not None:
        sub["stress"], sub["virials"] = out["stress"].cpu()[g], out["virials"].cpu()[g]
    return sub


def test_config2_full_batch_against_oracle_on_its_smallest_crystals():
    """Configuration 2: 64 random triclinic crystals, 89 elements, L = 3, 128 channels, r_cut 6.0, fp32.  The GPU
    evaluates the whole seed-1 batch; the oracle evaluates the five smallest crystals with the same 89-element weights."""
    wl = synth.WORKLOADS["crystals64_fp32"]
    structs = synth.workload_structures("crystals64_fp32")
    model, oracle, cfg = make_models(wl["L"], wl["channels"], wl["elements"], wl["cutoff"], wl["avg_num_neighbors"], torch.float32)
    data = oracle_batch(structs, wl["elements"], wl["cutoff"], torch.float32)
    out = model(to_device(data, DEV))
    torch.cuda.synchronize()
    assert model.device_error() == 0
    picks = sorted(np.argsort([len(s["positions"]) for s in structs], kind="stable")[:5].tolist())
    small = oracle_batch([structs[g] for g in picks], wl["elements"], wl["cutoff"], torch.float32)
    ref = oracle(small)
    check_parity(_subset(out, data, picks), ref, small["ptr"], torch.float32, "config 2 (89 elements, 5 smallest of 64 crystals)")


def test_config3_water_box_against_oracle():
    """Configuration 3's model (L = 3, 128 channels, r_cut 6.0, H and O, fp32) on a 64-molecule water box built by the
    same rules (rigid molecules on a jittered grid at 1.0 g/cm^3, random orientations, sigma 0.03 A)."""
    wl = synth.WORKLOADS["water32400_fp32"]
    box = 68.6 * (64 / 10800) ** (1.0 / 3.0)  # same density
    s = synth.water_box(n_side=4, box=box, sigma=0.03, seed=2, n_mol=64)
    model, oracle, cfg = make_models(wl["L"], wl["channels"], wl["elements"], wl["cutoff"], wl["avg_num_neighbors"], torch.float32,
                                     targets=("energy", "forces"))
    data = oracle_batch([s], wl["elements"], wl["cutoff"], torch.float32)
    assert data["edge_index"].shape[1] > 60 * 192  # cell (12.4 A) barely above twice the cutoff: about 90 neighbours per atom
    out = model(to_device(data, DEV))
    ref = oracle(data, compute_stress=False)
    check_parity(out, ref, data["ptr"], torch.float32, "config 3 (192-atom water box)")
    assert model.device_error() == 0


def test_config4_full_tece_model_against_oracle():
    """Configuration 4's model exactly (L = 3, 128 channels, 8 heads, edge_ace_hidden 32, element2 edge update, e3nn
    gate, identity skip, gated bilinear product, five elements, r_cut 6.0, fp32) on a 3 x 3 x 3 BCC cell."""
    wl = synth.WORKLOADS["tece8192_fp32"]
    s = synth.bcc_supercell(3, 2.87, 0.08, seed=3, species=tuple(wl["elements"]))
    model, oracle, cfg = make_models(wl["L"], wl["channels"], wl["elements"], wl["cutoff"], wl["avg_num_neighbors"], torch.float32,
                                     **wl["model"])
    data = oracle_batch([s], wl["elements"], wl["cutoff"], torch.float32)
    out = model(to_device(data, DEV))
    ref = oracle(data)
    check_parity(out, ref, data["ptr"], torch.float32, "config 4 (TECE, 54 atoms)")
    assert model.device_error() == 0


def test_config5_model_through_the_md_driver_against_oracle():
    """Configuration 5's model (L = 2, 64 channels, r_cut 5.0, Cu-Al, fp32) on a 4 x 4 x 4 FCC cell with 10 % Al,
    evaluated by the domain-decomposed MD driver on one rank (ghosts = periodic images), against the oracle."""
    from tace_b200.md import DomainMD

    wl = synth.WORKLOADS["cual1m_fp32"]
    s = synth.fcc_supercell(4, 3.65, 0.05, seed=4, species=(29, 13), fractions=(0.9, 0.1))
    model, oracle, cfg = make_models(wl["L"], wl["channels"], wl["elements"], wl["cutoff"], wl["avg_num_neighbors"], torch.float32,
                                     targets=("energy", "forces"))
    data = oracle_batch([s], wl["elements"], wl["cutoff"], torch.float32)
    ref = oracle(data, compute_stress=False)
    md = DomainMD(model.to(DEV), s["cell"], s["positions"], s["atomic_numbers"], skin=0.5, device=DEV)
    got = md.gather()
    n = len(s["positions"])
    de = abs(md.potential() - float(ref["energy"][0])) / n
    df = float(np.abs(got["forces"] - ref["forces"].double().numpy()).max())
    print(f"parity config 5 (256-atom Cu-Al through DomainMD) float32: dE_per_atom = {de:.3e}, dF = {df:.3e}")
    assert de <= 1e-5 and df <= 1e-4
    assert model.device_error() == 0


# ---- fixtures computed by the reference's own source files ----------------------------------------------------------
REFERENCE_FIXTURES = ["ref_model_cgtp_L2.npz", "ref_model_cgtp_L3_batch.npz", "ref_model_tece_L2_C32.npz",
                      "ref_model_options_a.npz", "ref_model_options_b.npz"]


def _load_fixture(name):
    z = np.load(os.path.join(GOLDEN, name), allow_pickle=False)
    cfg = json.loads(str(z["cfg_json"]))
    for s in cfg["statistics"]:  # JSON turned the integer keys of the per-element tables into strings
        for k, v in list(s.items()):
            if isinstance(v, dict):
                s[k] = {int(a): b for a, b in v.items()}
    zbl = cfg.get("short_range", {}).get("zbl", {})
    if "covalent_radii" in zbl:
        zbl["covalent_radii"] = {int(a): b for a, b in zbl["covalent_radii"].items()}
    sd = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("sd:")}
    data = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in:")}
    ref = {k[4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("out:")}
    return cfg, sd, data, ref


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name", REFERENCE_FIXTURES)
def test_cuda_path_reproduces_reference_source_outputs(name, dtype):
    """State dict, inputs and expected outputs all come from a run of the reference's own model code (fp64)."""
    cfg, sd, data, ref = _load_fixture(name)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        model = tace_b200.TensorModel(tace_b200.e3nnTACE(**cfg))
    finally:
        torch.set_default_dtype(prev)
    own = model.state_dict()
    model.load_state_dict({k: sd[k].to(own[k].dtype) for k in own})
    data = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in data.items()}
    out = model(to_device(data, DEV))
    check_parity(out, ref, data["ptr"], dtype, name)
    assert model.device_error() == 0
