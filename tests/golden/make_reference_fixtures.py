#!/usr/bin/env python
"""Writes ``tests/golden/ref_*.npz``: outputs of the REFERENCE's own source files, run in this container.

    python tests/golden/make_reference_fixtures.py          # needs the reference tree (TACE_REFERENCE_ROOT)

The reference's ``tace.models`` package is imported from its source tree by ``tests/refshim/loader.py``; the only
code on the evaluated path that is not the reference's is the stand-in for the third-party package e3nn
(``tests/refshim/mini_e3nn.py``: irreps bookkeeping, 3j symbols, harmonics, ``o3.Linear`` / ``o3.TensorProduct``
normalisation, ``Activation`` / gate plumbing - all taken from ``oracle/o3.py``).  So these fixtures pin the CPU oracle
against everything the reference implements itself - model assembly, path order, weight slicing, radial basis, ZBL,
scale / shift, derivatives, strain, the whole TECE edge block, LAMMPS ghost handling - and leave only the e3nn
conventions unpinned.  ``tests/test_oracle_vs_reference_sources.py`` compares the oracle with the stored values (and,
where the reference tree is present, re-runs the reference and compares that too).

Each model fixture holds: the model configuration (JSON), the state_dict (reference parameter names), the input
dictionary, and the reference's energy / node energy / forces / virials / stress (/ edge forces).
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

from helpers import oracle_batch  # noqa: E402
from refshim import loader  # noqa: E402
from tace_b200 import synth  # noqa: E402

ZBL_RADII = {1: 0.31, 8: 0.66, 13: 1.21, 29: 1.32}  # stand-in table shared by both sides (only ZBL reads it)


def reference_kwargs(cfg):
    """The reference's constructor has no defaults for these (hydra always passes the whole model section)."""
    full = json.loads(json.dumps(cfg))
    for k in ("node_embedding", "edge_embedding", "long_range", "universal_embedding"):
        full.setdefault(k, {})
    full.setdefault("fidelity", [{"name": f"f{i}", "atomic_energy": None} for i in range(len(cfg["statistics"]))])
    for s in full["statistics"]:  # JSON turned the integer keys of the per-element tables into strings
        for k, v in list(s.items()):
            if isinstance(v, dict):
                s[k] = {int(z): x for z, x in v.items()}
    zbl = full.get("short_range", {}).get("zbl", {})
    zbl.pop("covalent_radii", None)  # the reference reads ase.data.covalent_radii (the stand-in table holds ZBL_RADII)
    return full


def perturb_(sd, seed):
    """The reference initialises biases, the attention's radial projection and the density offset to zero and the
    element-dependent edge update to 1e-3; move them away so that every term matters (the rules of tests/helpers.py)."""
    g = torch.Generator().manual_seed(seed + 1)
    for k, v in sd.items():
        if not v.is_floating_point():
            continue
        if k.endswith(".bias"):
            v.copy_(0.3 * torch.randn(v.shape, generator=g, dtype=v.dtype))
        if ".edge_info.mlp." in k and k.endswith(".weight") and v.dim() == 1:
            v.copy_(1.0 + 0.3 * torch.randn(v.shape, generator=g, dtype=v.dtype))
        if "radial_proj.weight" in k or ".edge_updates." in k:
            v.copy_(torch.randn(v.shape, generator=g, dtype=v.dtype))
        if k.endswith(".beta"):
            v.copy_(torch.tensor(0.8, dtype=v.dtype))
        if k.endswith(".alpha"):
            v.copy_(torch.tensor(3.0 + torch.rand((), generator=g).item(), dtype=v.dtype))
    sd["readout_fn.scale_shift.scale"].copy_(0.5 + torch.rand(sd["readout_fn.scale_shift.scale"].shape, generator=g))
    sd["readout_fn.atomic_energy_layer.atomic_energy"].copy_(
        torch.randn(sd["readout_fn.atomic_energy_layer.atomic_energy"].shape, generator=g))
    return sd


def build_reference(cfg, state_dict=None, seed=0):
    tm = loader.load(covalent_radii=covalent_table())
    torch.manual_seed(seed)
    model = tm.TensorModel(tm.e3nnTACE(**reference_kwargs(cfg)))
    if state_dict is None:  # weights rounded to fp32 so that the fixture can store them in half the space
        sd = perturb_(model.state_dict(), seed)
        model.load_state_dict({k: (v.float().double() if v.is_floating_point() else v) for k, v in sd.items()}, strict=True)
        return model
    own = model.state_dict()
    missing = [k for k in own if k not in state_dict]
    extra = [k for k in state_dict if k not in own]
    assert not missing and not extra, (missing[:5], extra[:5])
    model.load_state_dict({k: state_dict[k].to(own[k].dtype) for k in own}, strict=True)
    return model


def covalent_table():
    table = np.full(119, 0.2)
    for z, r in ZBL_RADII.items():
        table[z] = r
    return table


def run_reference(model, data):
    out = model({k: (v.clone() if torch.is_tensor(v) else v) for k, v in data.items()})
    return {k: v.detach() for k, v in out.items() if torch.is_tensor(v)}


def save(name, cfg, sd, data, out, extra=None):
    arrays = {"cfg_json": np.array(json.dumps(cfg))}
    arrays.update({"sd:" + k: (v.detach().float().numpy() if v.is_floating_point() else v.numpy()) for k, v in sd.items()})
    assert all(torch.equal(v.float().double(), v.double()) for v in sd.values() if v.is_floating_point())
    arrays.update({"in:" + k: v.numpy() for k, v in data.items() if torch.is_tensor(v)})
    arrays.update({"out:" + k: v.numpy() for k, v in out.items()})
    arrays.update(extra or {})
    np.savez_compressed(os.path.join(HERE, name), **arrays)
    print(f"{name}: {os.path.getsize(os.path.join(HERE, name)) / 1024:.0f} KiB,", {k: tuple(v.shape) for k, v in out.items()})


def retype(structures, elements):
    """Random crystals draw species from Z = 1..89; map them onto the few elements of a small test model."""
    for s in structures:
        s["atomic_numbers"] = np.asarray([elements[int(z) % len(elements)] for z in s["atomic_numbers"]], dtype=np.int64)
    return structures


MODEL_CASES = {
    # BASELINE configuration 1 at reduced width: cgtp, L = 2, one element, FCC
    "ref_model_cgtp_L2.npz": dict(structures=lambda: [synth.fcc_supercell(2, 3.61, 0.05, seed=0)], elements=[29], cutoff=4.0,
                                  model=dict(L=2, C=16)),
    # configuration 2 / 3 shape: L = 3, several elements, a batch of triclinic crystals with self images
    "ref_model_cgtp_L3_batch.npz": dict(structures=lambda: retype(synth.random_crystals(3, seed=7, nmin=3, nmax=6), [1, 8, 29]), elements=[1, 8, 29],
                                        cutoff=4.5, model=dict(L=3, C=8)),
    # configuration 4: the reference's example TECE model section (element2 edge update, bias, e3nn Gate, identity
    # skip, gated bilinear product with one coefficient matrix for all species, uv_so2 second layer)
    "ref_model_tece_L3.npz": dict(structures=lambda: [synth.bcc_supercell(2, 2.87, 0.08, seed=3, species=(26, 28))], elements=[26, 28],
                                  cutoff=4.0,
                                  model=dict(L=3, C=8, gate_m0=False, edge_update="element2",
                                             radial={"apply_cutoff": False, "bias": True, "hidden": [64, 64]},
                                             resnet_linear_type="identity", product_agnostic=True,
                                             product_nonlinear="silu_bilineargate",
                                             tece={"num_head": 2, "edge_ace_hidden": 4, "mmax": 2})),
    # TECE block with its defaults on a plain model (sigmoid gates everywhere, envelope inside the features)
    "ref_model_tece_L2_plain.npz": dict(structures=lambda: [synth.bcc_supercell(2, 2.87, 0.08, seed=3, species=(26, 28))],
                                        elements=[26, 28], cutoff=4.0,
                                        model=dict(L=2, C=8, radial={"apply_cutoff": False},
                                                   tece={"num_head": 4, "edge_ace_hidden": 8, "mmax": 2})),
    # the same block at a channel count the CUDA kernels take (multiples of 32), for the GPU tests
    "ref_model_tece_L2_C32.npz": dict(structures=lambda: [synth.bcc_supercell(2, 2.87, 0.08, seed=3, species=(26, 28))],
                                      elements=[26, 28], cutoff=4.0,
                                      model=dict(L=2, C=32, radial={"apply_cutoff": False},
                                                 tece={"num_head": 4, "edge_ace_hidden": 8, "mmax": 2})),
    # options: correlation 3, read-outs of all layers, ZBL, node rank below edge rank
    "ref_model_options_a.npz": dict(structures=lambda: [synth.fcc_supercell(2, 3.61, 0.05, seed=1, species=(13, 29), fractions=(0.3, 0.7))], elements=[13, 29],
                                    cutoff=4.0,
                                    model=dict(L=3, Lmax=2, C=8, correlation=3, use_alllayer=True,
                                               zbl={"enable": True, "covalent_radii": ZBL_RADII}, scale_zbl=False)),
    # options: e3nn Gate, learned edge density, two fidelities, three layers
    "ref_model_options_b.npz": dict(structures=lambda: retype(synth.random_crystals(2, seed=11, nmin=3, nmax=5), [1, 8]), elements=[1, 8], cutoff=4.0,
                                    model=dict(L=2, C=8, num_layers=3, gate_m0=False, scatter_norm="density", num_fidelities=2),
                                    fidelity_idx=[1, 0]),
}


def model_cases():
    for name, case in MODEL_CASES.items():
        kw = dict(case["model"])
        cfg = synth.model_config(kw.pop("L"), kw.pop("C"), case["cutoff"], case["elements"], 20.0, **kw)
        ref = build_reference(cfg)
        sd = ref.state_dict()
        data = oracle_batch(case["structures"](), case["elements"], case["cutoff"], torch.float64)
        if "fidelity_idx" in case:
            data["fidelity_idx"] = torch.tensor(case["fidelity_idx"], dtype=torch.int64)
        out = run_reference(ref, data)
        save(name, cfg, sd, data, out)


def lammps_case():
    """The reference in LAMMPS mode (``tace/models/lammps.py``, ``tace/interface/lammps/mliap.py:25-52``): owned atoms of
    a periodic cell plus ghost images, features refreshed / gradients returned through a fake ``lmp_data`` that follows
    the ML-IAP exchange contract.  Stored: per-pair dE/d(edge vector), owned-atom energies, and the ghost -> owner map."""
    structure = synth.fcc_supercell(2, 3.61, 0.05, seed=2, species=(13, 29), fractions=(0.3, 0.7))
    elements, cutoff = [13, 29], 4.0
    cfg = synth.model_config(2, 8, cutoff, elements, 20.0, target_property=("energy", "forces"))
    ref = build_reference(cfg)
    sd = ref.state_dict()
    periodic = oracle_batch([structure], elements, cutoff, torch.float64)
    n = periodic["positions"].shape[0]
    src, dst = periodic["edge_index"]
    shifts = periodic["edge_shifts"]
    ghost_of, owner = {}, []
    local_src = src.clone()
    for e in range(src.numel()):
        key = (int(src[e]),) + tuple(int(x) for x in shifts[e])
        if any(key[1:]):
            if key not in ghost_of:
                ghost_of[key] = n + len(owner)
                owner.append(int(src[e]))
            local_src[e] = ghost_of[key]
    owner = torch.tensor(owner, dtype=torch.int64)
    pos, cell = periodic["positions"], periodic["lattice"][0]
    edge_vector = pos[dst] - pos[src] + shifts @ cell  # the reference's own convention: target - source
    node_attrs = torch.cat([periodic["node_attrs"], periodic["node_attrs"][owner]])

    class FakeLammpsData:
        def forward_exchange(self, src_rows, out_rows, vec_len):
            out_rows.copy_(src_rows)
            out_rows[n:] = src_rows[owner]

        def reverse_exchange(self, grad_rows, out_rows, vec_len):
            out_rows.copy_(grad_rows)
            out_rows[:n].index_add_(0, owner, grad_rows[n:])
            out_rows[n:] = 0

    ref.lmp = True
    ref.flags.compute_forces = False
    ref.flags.compute_stress = False
    ref.flags.compute_virials = False
    ref.flags.compute_edge_forces = True
    data = {"edge_vector": edge_vector.clone(), "node_attrs": node_attrs, "edge_index": torch.stack([local_src, dst]),
            "batch": torch.zeros(n, dtype=torch.int64), "ptr": torch.tensor([0, n]), "lmp_data": FakeLammpsData(),
            "natoms": (n, int(owner.numel()))}
    out = ref(data)
    out = {k: v.detach() for k, v in out.items() if torch.is_tensor(v) and k in ("energy", "node_energy", "edge_forces")}
    tensors = {k: v for k, v in data.items() if torch.is_tensor(v)}
    tensors["edge_vector"] = edge_vector
    extra = {"per:" + k: v.numpy() for k, v in periodic.items()}
    extra["ghost_owner"] = owner.numpy()
    save("ref_model_lammps_L2.npz", cfg, sd, tensors, out, extra)


def component_cases():
    """Single functions / modules of the reference, on seeded fp64 inputs."""
    tm = loader.load(covalent_radii=covalent_table())
    import importlib

    g = torch.Generator().manual_seed(5)
    out = {}
    # --- edge frame and Wigner rows (tace/models/o2/rotation_matrix.py:74-88, tace/models/o2/wigner.py:178-357)
    rot = importlib.import_module("tace.models.o2.rotation_matrix")
    wig = importlib.import_module("tace.models.o2.wigner")
    vec = torch.randn(40, 3, generator=g, dtype=torch.float64) * 2.0
    vec[0] = torch.tensor([0.0, 1.0, 0.0])
    vec[1] = torch.tensor([0.0, -1.0, 0.0])
    vec[2] = torch.tensor([1e-4, -1.0, 2e-4])
    vec[3] = torch.tensor([1e-4, 1.0, -2e-4])
    vec[4] = torch.tensor([0.3, 0.0, -0.4])
    out["frame_vectors"] = vec
    out["frame_rotation"] = rot.init_edge_rot_mat_quaternion(vec)
    for lmax, mmax in ((3, 2), (2, 2), (3, 1), (2, 1)):
        w = wig.WignerD(mmax, lmax)
        a, b = w.get_wigner(vec)
        out[f"wigner_l{lmax}_m{mmax}"], out[f"wigner_inv_l{lmax}_m{mmax}"] = a, b
    # --- segment softmax with rescale (tace/models/softmax.py:80-114)
    sm = importlib.import_module("tace.models.softmax")
    logits = torch.randn(30, 4, generator=g, dtype=torch.float64) * 3
    index = torch.randint(0, 6, (30,), generator=g)
    index[index == 4] = 3  # an empty segment
    rescale = torch.rand(30, 1, generator=g, dtype=torch.float64)
    out["softmax_logits"], out["softmax_index"], out["softmax_rescale"] = logits, index, rescale
    out["softmax_out"] = sm.GraphSoftmax()(logits, index, num_nodes=6, exp_rescale=rescale)
    out["softmax_out_plain"] = sm.GraphSoftmax()(logits, index, num_nodes=6)
    # --- radial basis, envelope, ZBL (tace/models/radial.py:43-84,437-472,788-874,877-993)
    radial = importlib.import_module("tace.models.radial")
    r = torch.cat([torch.linspace(0.4, 5.3, 50, dtype=torch.float64), torch.tensor([4.999999, 5.0, 5.000001], dtype=torch.float64)]).unsqueeze(-1)
    out["radial_r"] = r
    out["radial_j0"] = radial.j0SphericalBesselBasis(cutoff=5.0, num_basis=8)(r, None, None)
    out["radial_c2poly"] = radial.C2PolynomialCutoff(cutoff=5.0, p=5)(r)
    # --- radial MLP (tace/models/mlp.py:136-191, tace/models/linear.py:247-279)
    mlp_mod = importlib.import_module("tace.models.mlp")
    torch.manual_seed(3)
    for tag, kw in (("plain", {}), ("bias_ln", {"bias": True, "layer_norm": True})):
        mlp = mlp_mod.MLP([8, 64, 64, 24], **kw)
        for name, p in mlp.named_parameters():
            if p.dim() == 1:  # biases and LayerNorm scales away from their initial 0 / 1
                p.data.copy_((1.0 if name.endswith("weight") else 0.0) + 0.2 * torch.randn(p.shape, generator=g, dtype=p.dtype))
        x = torch.randn(11, 8, generator=g, dtype=torch.float64)
        out[f"mlp_{tag}_in"] = x
        out[f"mlp_{tag}_out"] = mlp(x).detach()
        for k, v in mlp.state_dict().items():
            out[f"mlp_{tag}_sd:{k}"] = v
    # --- strain / virial / stress helpers (tace/models/utils.py:50-115) are exercised by every model case with stress
    np.savez_compressed(os.path.join(HERE, "ref_components.npz"), **{k: v.detach().numpy() for k, v in out.items()})
    print("ref_components.npz:", sorted(out))


def main():
    if not loader.available():
        sys.exit("the reference tree is not available; fixtures can only be regenerated where it is")
    torch.set_default_dtype(torch.float64)
    component_cases()
    model_cases()
    lammps_case()


if __name__ == "__main__":
    main()
