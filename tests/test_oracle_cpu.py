"""The oracle against the golden vectors, the reference-held constants, and its own invariances."""
import os

import numpy as np
import torch

from oracle import o3
from oracle.model import build_oracle
from oracle.neighbour_list import neighbour_list
from golden_util import GOLDEN, load_case
from helpers import oracle_batch


def test_activation_constants_match_the_reference():
    """tace/models/mlp.py:34,43,52, pinned by the reference's tests/test_o2.py:352-376."""
    ref = np.load(os.path.join(GOLDEN, "o3_tables.npz"))["activation_constants_reference"]
    got = [o3.second_moment_constant(n) for n in ("silu", "sigmoid", "tanh")]
    np.testing.assert_allclose(got, ref, rtol=0, atol=1e-12)


def test_o3_tables_match_golden_and_are_consistent():
    tab = np.load(os.path.join(GOLDEN, "o3_tables.npz"))
    for key in tab.files:
        if key.startswith("w3j_"):
            l1, l2, l3 = (int(c) for c in key[4:])
            w = o3.wigner_3j(l1, l2, l3).numpy()
            np.testing.assert_allclose(w, tab[key], rtol=0, atol=1e-14)
            assert abs(np.linalg.norm(w) - 1.0) < 1e-12
    pts = torch.from_numpy(tab["sh_points"])
    np.testing.assert_allclose(o3.spherical_harmonics(3, pts, "component").numpy(), tab["sh_values_component"], atol=1e-14)
    # documented special cases of the real basis: (1,1,1) is the Levi-Civita tensor / sqrt(6), (l,l,0) the identity
    eps = np.zeros((3, 3, 3))
    for i, j, k in [(0, 1, 2), (1, 2, 0), (2, 0, 1)]:
        eps[i, j, k], eps[i, k, j] = 1.0, -1.0
    np.testing.assert_allclose(o3.wigner_3j(1, 1, 1).numpy(), eps / np.sqrt(6), atol=1e-14)
    for l in range(4):
        np.testing.assert_allclose(o3.wigner_3j(l, l, 0).numpy()[:, :, 0], np.eye(2 * l + 1) / np.sqrt(2 * l + 1), atol=1e-14)


def test_cartesian_tensors_match_spherical_harmonics():
    """The reference's Cartesian route (tace/models/angular.py:52-90): symmetric traceless part of n (x) n and
    n (x) n (x) n has squared norm (2l-1)!!/l! and carries the same information as the l-th harmonics."""
    torch.manual_seed(0)
    n = torch.randn(3, dtype=torch.float64)
    n = n / n.norm()
    t2 = torch.outer(n, n) - torch.eye(3, dtype=torch.float64) / 3.0
    assert abs((t2**2).sum().item() * (3.0 / 2.0) ** 2 - 1.5) < 1e-12  # ((2l-1)!!/l!) STF(n n) has |.|^2 = 3/2
    Y = o3.spherical_harmonics(2, n[None], "norm")[0, 4:9]
    # |Y_2|^2 = 1 and Y_2 is linear in the five independent components of t2
    assert abs((Y**2).sum().item() - 1.0) < 1e-12
    x, y, z = n
    np.testing.assert_allclose(Y[2].item(), 1.5 * t2[1, 1].item(), atol=1e-12)
    np.testing.assert_allclose(Y[0].item(), np.sqrt(3.0) * t2[0, 2].item(), atol=1e-12)


def test_oracle_reproduces_golden_model_case():
    blob, sd, cfg, s = load_case()
    oracle = build_oracle(cfg, sd, torch.float64)
    data = oracle_batch([s], [29], float(blob["cutoff"]), torch.float64)
    assert np.array_equal(data["edge_index"].numpy(), blob["edge_index"])
    ref = oracle(data)
    np.testing.assert_allclose(ref["energy"].numpy(), blob["energy"], rtol=0, atol=1e-9)
    np.testing.assert_allclose(ref["forces"].numpy(), blob["forces"], rtol=0, atol=1e-10)
    np.testing.assert_allclose(ref["stress"].numpy(), blob["stress"], rtol=0, atol=1e-10)


def test_oracle_reproduces_golden_tece_case():
    """The stored case with the TECE edge block (tests/golden/case_bcc16_tece_L2_C32.npz)."""
    blob, sd, cfg, s = load_case("case_bcc16_tece_L2_C32.npz")
    oracle = build_oracle(cfg, sd, torch.float64)
    ref = oracle(oracle_batch([s], [int(z) for z in blob["elements"]], float(blob["cutoff"]), torch.float64))
    np.testing.assert_allclose(ref["energy"].numpy(), blob["energy"], rtol=0, atol=1e-9)
    np.testing.assert_allclose(ref["forces"].numpy(), blob["forces"], rtol=0, atol=1e-10)
    np.testing.assert_allclose(ref["stress"].numpy(), blob["stress"], rtol=0, atol=1e-10)


def test_oracle_neighbour_list_golden():
    g = np.load(os.path.join(GOLDEN, "neighbour_list_triclinic5.npz"))
    ei, es = neighbour_list(g["positions"], g["cell"], (True, True, True), float(g["cutoff"]))
    assert np.array_equal(ei, g["edge_index"]) and np.array_equal(es, g["edge_shifts"])
    # full list: every edge has its reverse, self images are present (cell narrower than the cutoff)
    fwd = {(int(a), int(b), *map(int, s)) for (a, b), s in zip(ei.T, es)}
    assert all((b, a, -x, -y, -z) in fwd for (a, b, x, y, z) in fwd)
    assert any(a == b for (a, b, *_s) in fwd)


def test_oracle_invariances():
    """Rotation / translation invariance of E, equivariance of F, sum of forces zero, F vs finite differences."""
    blob, sd, cfg, s = load_case()
    oracle = build_oracle(cfg, sd, torch.float64)
    base = oracle(oracle_batch([s], [29], 4.0, torch.float64))
    assert base["forces"].sum(0).abs().max().item() < 1e-10
    q, _ = np.linalg.qr(np.random.default_rng(0).normal(size=(3, 3)))
    rot = dict(s)
    rot["positions"] = s["positions"] @ q.T + np.array([0.3, -0.2, 0.1]) @ (s["cell"] @ q.T)
    rot["cell"] = s["cell"] @ q.T
    r = oracle(oracle_batch([rot], [29], 4.0, torch.float64))
    assert abs(r["energy"].item() - base["energy"].item()) < 1e-9
    np.testing.assert_allclose(r["forces"].numpy(), base["forces"].numpy() @ q.T, atol=1e-9)
    h = 1e-5
    for (i, k) in [(0, 0), (5, 2)]:
        e = []
        for sign in (+1, -1):
            p = dict(s)
            p["positions"] = s["positions"].copy()
            p["positions"][i, k] += sign * h
            e.append(oracle(oracle_batch([p], [29], 4.0, torch.float64))["energy"].item())
        fd = -(e[0] - e[1]) / (2 * h)
        assert abs(fd - base["forces"][i, k].item()) < 1e-6
