"""Pins the CPU oracle against the reference's own source files.

``tests/golden/ref_*.npz`` were written by ``tests/golden/make_reference_fixtures.py``, which imports the reference's
``tace.models`` package from its source tree (third-party packages replaced by the stand-ins of ``tests/refshim``) and
stores what the reference's code computes.  Here the oracle gets the same configuration, state_dict and inputs and has
to reproduce those numbers to fp64 round-off.  Where the reference tree is present the reference is also re-run, so the
fixtures cannot drift from the sources.  What stays unpinned is exactly what the stand-in for e3nn supplies from
``oracle/o3.py``: 3j symbols, spherical harmonics, TensorProduct / Linear normalisation, activation constants.
"""
import json
import os

import numpy as np
import pytest
import torch

from oracle import tece as oracle_tece
from oracle.model import MLP, C2Poly, J0Bessel, build_oracle, scatter_sum
from refshim import loader

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 1e-10  # relative to max(1, largest reference entry); fp64 round-off through softmax and LayerNorm reaches 1e-11

MODEL_FIXTURES = ["ref_model_cgtp_L2.npz", "ref_model_cgtp_L3_batch.npz", "ref_model_tece_L3.npz",
                  "ref_model_tece_L2_plain.npz", "ref_model_tece_L2_C32.npz", "ref_model_options_a.npz",
                  "ref_model_options_b.npz"]


def _close(a, b, what, tol=TOL):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    err = np.abs(a - b).max() if a.size else 0.0
    scale = max(1.0, np.abs(b).max() if b.size else 0.0)
    assert err <= tol * scale, f"{what}: max abs deviation {err:.3e} (scale {scale:.3e})"


def _load(name):
    z = np.load(os.path.join(GOLDEN, name), allow_pickle=False)
    cfg = json.loads(str(z["cfg_json"]))
    for s in cfg["statistics"]:
        for k, v in list(s.items()):
            if isinstance(v, dict):
                s[k] = {int(a): b for a, b in v.items()}
    zbl = cfg.get("short_range", {}).get("zbl", {})
    if "covalent_radii" in zbl:
        zbl["covalent_radii"] = {int(a): b for a, b in zbl["covalent_radii"].items()}
    sd = {k[3:]: torch.from_numpy(z[k].astype(np.float64) if z[k].dtype == np.float32 else z[k]) for k in z.files if k.startswith("sd:")}
    data = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("in:")}
    out = {k[4:]: z[k] for k in z.files if k.startswith("out:")}
    return z, cfg, sd, data, out


@pytest.mark.parametrize("name", MODEL_FIXTURES)
def test_oracle_reproduces_reference_model_outputs(name):
    _, cfg, sd, data, ref = _load(name)
    oracle = build_oracle(cfg, sd, torch.float64)
    out = oracle(data)
    # ZBL pair terms are thousands of eV before the envelope cuts them down: their round-off sets a coarser floor
    tol = 1e-9 if cfg["short_range"]["zbl"].get("enable") else TOL
    for key in ("energy", "node_energy", "forces", "virials", "stress"):
        _close(out[key], ref[key], f"{name}:{key}", tol)


def test_oracle_reproduces_reference_lammps_mode():
    """Reference: owned + ghost atoms, ghost rows refreshed after layer 0, gradients returned to the owners
    (tace/models/lammps.py:82-142).  Oracle: the same periodic cell evaluated as one graph."""
    z, cfg, sd, data, ref = _load("ref_model_lammps_L2.npz")
    periodic = {k[4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("per:")}
    oracle = build_oracle(cfg, sd, torch.float64)
    out = oracle(periodic, compute_stress=False, compute_edge_forces=True)
    n = periodic["positions"].shape[0]
    _close(out["node_energy"], ref["node_energy"][:n], "node_energy")
    _close(out["energy"][0], ref["energy"][0], "energy")
    _close(out["edge_forces"], ref["edge_forces"], "edge_forces")
    # pair forces of the reference assemble to the oracle's forces: F_i = sum_{e: src=i} g_e - sum_{e: dst=i} g_e
    g = torch.from_numpy(ref["edge_forces"])
    src, dst = periodic["edge_index"]
    f = scatter_sum(g, src, n) - scatter_sum(g, dst, n)
    _close(f, out["forces"], "forces from pair forces")


def test_edge_frame_and_wigner_rows_match_reference():
    z = np.load(os.path.join(GOLDEN, "ref_components.npz"))
    vec = torch.from_numpy(z["frame_vectors"])
    _close(oracle_tece.edge_rotation(vec), z["frame_rotation"], "edge frame")
    for lmax, mmax in ((3, 2), (2, 2), (3, 1), (2, 1)):
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.float64)  # the rescale constants are built in the default dtype
        try:
            w, winv = oracle_tece.WignerD(mmax, lmax).get_wigner(vec)
        finally:
            torch.set_default_dtype(prev)
        _close(w, z[f"wigner_l{lmax}_m{mmax}"], f"wigner rows l{lmax} m{mmax}")
        _close(winv, z[f"wigner_inv_l{lmax}_m{mmax}"], f"inverse wigner rows l{lmax} m{mmax}")


def test_segment_softmax_matches_reference():
    z = np.load(os.path.join(GOLDEN, "ref_components.npz"))
    logits, index = torch.from_numpy(z["softmax_logits"]), torch.from_numpy(z["softmax_index"])
    out = oracle_tece.graph_softmax(logits, index, 6, exp_rescale=torch.from_numpy(z["softmax_rescale"]))
    _close(out, z["softmax_out"], "softmax with rescale")
    _close(oracle_tece.graph_softmax(logits, index, 6), z["softmax_out_plain"], "softmax")


def test_radial_basis_and_mlp_match_reference():
    z = np.load(os.path.join(GOLDEN, "ref_components.npz"))
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.float64)
    try:
        r = torch.from_numpy(z["radial_r"])
        _close(J0Bessel(5.0, 8)(r), z["radial_j0"], "bessel basis")
        _close(C2Poly(5.0, 5)(r), z["radial_c2poly"], "polynomial cutoff")
        for tag, kw in (("plain", {}), ("bias_ln", {"bias": True, "layer_norm": True})):
            mlp = MLP([8, 64, 64, 24], **kw)
            sd = {k.split(":", 1)[1]: torch.from_numpy(z[k]) for k in z.files if k.startswith(f"mlp_{tag}_sd:")}
            mlp.load_state_dict(sd, strict=True)
            _close(mlp(torch.from_numpy(z[f"mlp_{tag}_in"])).detach(), z[f"mlp_{tag}_out"], f"radial MLP ({tag})")
    finally:
        torch.set_default_dtype(prev)


# ---- live half: only where the reference tree exists ------------------------------------------------------------
needs_reference = pytest.mark.skipif(not loader.available(), reason="the reference source tree is not on this machine")


@needs_reference
@pytest.mark.parametrize("name", MODEL_FIXTURES)
def test_fixture_is_what_the_reference_sources_compute(name):
    import sys

    sys.path.insert(0, GOLDEN)
    import make_reference_fixtures as gen

    _, cfg, sd, data, ref = _load(name)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.float64)
    try:
        out = gen.run_reference(gen.build_reference(cfg, sd), data)
    finally:
        torch.set_default_dtype(prev)
    for key in ("energy", "node_energy", "forces", "virials", "stress"):
        _close(out[key], ref[key], f"{name}:{key} (live reference)", tol=1e-13)


@needs_reference
def test_state_dict_names_are_the_reference_s():
    """Every fixture's parameter names come from the reference model's own ``state_dict()``; the oracle and the CUDA
    model's packer must accept exactly those."""
    import sys

    sys.path.insert(0, GOLDEN)
    import make_reference_fixtures as gen

    for name in MODEL_FIXTURES:
        _, cfg, sd, _, _ = _load(name)
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.float64)
        try:
            ref_keys = set(gen.build_reference(cfg, sd).state_dict())
            oracle_keys = set(build_oracle(cfg, sd, torch.float64).state_dict())
        finally:
            torch.set_default_dtype(prev)
        assert ref_keys == set(sd), name
        assert oracle_keys <= ref_keys, (name, sorted(oracle_keys - ref_keys)[:5])
