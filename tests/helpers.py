"""Shared helpers of the parity tests: build matching CUDA / oracle models and inputs."""
from __future__ import annotations

import numpy as np
import torch

import tace_b200
from tace_b200 import synth


def make_models(L, C, elements, cutoff, avg, dtype, seed=0, num_layers=2, correlation=2,
                targets=("energy", "forces", "stress"), Lmax=None, use_alllayer=False, gate_m0=True, radial=None, edge_update="identity",
                num_fidelities=1, zbl=None, scale_zbl=True, scatter_norm="avg_num_neighbors",
                resnet_linear_type="aware", product_agnostic=False, product_nonlinear=None, tece=None):
    """The CUDA-backed TensorModel and the CPU oracle sharing one seeded state_dict."""
    from oracle.model import build_oracle

    cfg = synth.model_config(L, C, cutoff, elements, avg, num_layers=num_layers, correlation=correlation,
                             target_property=targets, Lmax=Lmax, use_alllayer=use_alllayer, gate_m0=gate_m0, radial=radial, edge_update=edge_update,
                             num_fidelities=num_fidelities, zbl=zbl, scale_zbl=scale_zbl, scatter_norm=scatter_norm,
                             resnet_linear_type=resnet_linear_type, product_agnostic=product_agnostic,
                             product_nonlinear=product_nonlinear, tece=tece)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        torch.manual_seed(seed)
        model = tace_b200.TensorModel(tace_b200.e3nnTACE(**cfg))
        # non-zero biases and species-dependent scale / E0 so every term is exercised
        g = torch.Generator().manual_seed(seed + 1)
        sd = model.state_dict()
        for k, v in sd.items():
            if k.endswith(".bias"):
                v.copy_(0.3 * torch.randn(v.shape, generator=g, dtype=v.dtype))
            if ".edge_info.mlp." in k and k.endswith(".weight") and v.dim() == 1:  # LayerNorm scale: away from 1
                v.copy_(1.0 + 0.3 * torch.randn(v.shape, generator=g, dtype=v.dtype))
            if "radial_proj.weight" in k:  # zero in the reference's initialisation: make the radial bias and phase matter
                v.copy_(torch.randn(v.shape, generator=g, dtype=v.dtype))
            if k.endswith(".beta"):  # zero in the reference's initialisation: switch the learned density on
                v.copy_(torch.tensor(0.8, dtype=v.dtype))
            if k.endswith(".alpha"):
                v.copy_(torch.tensor(3.0 + torch.rand((), generator=g).item(), dtype=v.dtype))
            if ".edge_updates." in k:  # initialised at 1e-3 in the reference: make the term visible
                v.copy_(torch.randn(v.shape, generator=g, dtype=v.dtype))
        sd["readout_fn.scale_shift.scale"].copy_(0.5 + torch.rand(sd["readout_fn.scale_shift.scale"].shape, generator=g, dtype=dtype))
        sd["readout_fn.atomic_energy_layer.atomic_energy"].copy_(
            torch.randn(sd["readout_fn.atomic_energy_layer.atomic_energy"].shape, generator=g, dtype=dtype))
    finally:
        torch.set_default_dtype(prev)
    oracle = build_oracle(cfg, model.state_dict(), dtype)
    return model, oracle, cfg


def oracle_batch(structures, elements, cutoff, dtype):
    """Input dictionary for the oracle with the brute-force neighbour list (CPU tensors)."""
    from oracle.neighbour_list import neighbour_list

    b = synth.collate(structures)
    eis, ess = [], []
    for s, off in zip(structures, b["ptr"][:-1]):
        ei, es = neighbour_list(s["positions"], s["cell"], s["pbc"], cutoff)
        eis.append(ei + off)
        ess.append(es)
    zs = sorted(elements)
    idx = np.array([zs.index(int(z)) for z in b["atomic_numbers"]])
    return {
        "positions": torch.tensor(b["positions"], dtype=dtype),
        "lattice": torch.tensor(b["lattice"], dtype=dtype),
        "node_attrs": torch.nn.functional.one_hot(torch.tensor(idx), len(zs)).to(dtype),
        "edge_index": torch.tensor(np.concatenate(eis, axis=1), dtype=torch.int64),
        "edge_shifts": torch.tensor(np.concatenate(ess, axis=0), dtype=dtype),
        "batch": torch.tensor(b["batch"]),
        "ptr": torch.tensor(b["ptr"]),
    }


def to_device(data, device):
    return {k: v.to(device) for k, v in data.items()}


def feats_to_oracle_layout(x: torch.Tensor, ls, C: int) -> torch.Tensor:
    """[n][component][channel] (rank blocks in `ls`) -> e3nn mul_ir [n][sum_l C*(2l+1)]."""
    n = x.shape[0]
    x = x.reshape(n, -1, C)
    out, off = [], 0
    for l in ls:
        blk = x[:, off:off + 2 * l + 1, :]  # [n, m, c]
        out.append(blk.permute(0, 2, 1).reshape(n, -1))
        off += 2 * l + 1
    return torch.cat(out, dim=1)


# The task's tolerances, absolute: fp64 energy 1e-8 eV/atom, forces 1e-7 eV/A; fp32 1e-5 eV/atom, 1e-4 eV/A.
PARITY_TOL = {torch.float64: (1e-8, 1e-7), torch.float32: (1e-5, 1e-4)}


def check_parity(out, ref, ptr, dtype, label=""):
    """Asserts the absolute tolerances and prints the worst deviations (shown by ``pytest -s`` / on failure).

    Energy per atom and forces carry the stated absolute bounds.  Per-atom energies get ten times the energy bound,
    stress the force bound (eV/A^3).  Virials are extensive (a sum of r x F over all edges of a graph), so their bound
    is the force bound times max(1, largest reference entry).  Returns the deviations."""
    etol, ftol = PARITY_TOL[dtype]
    n_per_graph = (ptr[1:] - ptr[:-1]).to(torch.float64).cpu()
    cpu = lambda t: t.detach().cpu().to(torch.float64)
    dev = {"dE_per_atom": ((cpu(out["energy"]) - cpu(ref["energy"])).abs() / n_per_graph).max().item(),
           "dF": (cpu(out["forces"]) - cpu(ref["forces"])).abs().max().item() if ref.get("forces") is not None else 0.0}
    if ref.get("node_energy") is not None and out.get("node_energy") is not None:
        dev["dE_node"] = (cpu(out["node_energy"]) - cpu(ref["node_energy"])).abs().max().item()
    if ref.get("stress") is not None and out.get("stress") is not None:
        dev["dStress"] = (cpu(out["stress"]) - cpu(ref["stress"])).abs().max().item()
        dev["dVirial"] = (cpu(out["virials"]) - cpu(ref["virials"])).abs().max().item()
    print(f"parity {label} {str(dtype).replace('torch.', '')}: " + ", ".join(f"{k} = {v:.3e}" for k, v in dev.items()))
    assert dev["dE_per_atom"] <= etol, f"{label}: |dE|/atom = {dev['dE_per_atom']:.3e} eV > {etol}"
    assert dev["dF"] <= ftol, f"{label}: max |dF| = {dev['dF']:.3e} eV/A > {ftol}"
    if "dE_node" in dev:
        assert dev["dE_node"] <= 10 * etol, f"{label}: per-atom energy deviates by {dev['dE_node']:.3e} eV"
    if "dStress" in dev:
        assert dev["dStress"] <= ftol, f"{label}: stress deviates by {dev['dStress']:.3e} eV/A^3"
        vmax = max(1.0, cpu(ref["virials"]).abs().max().item())
        assert dev["dVirial"] <= ftol * vmax, f"{label}: virial deviates by {dev['dVirial']:.3e} eV (largest entry {vmax:.3e})"
    return dev
