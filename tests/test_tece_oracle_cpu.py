"""Internal-consistency pins of the TECE edge block restatement (oracle/tece.py), CPU only.

The reference cannot run here, so these tests pin what can be pinned without it: the Wigner matrices built by the
reference's recursion rotate this package's spherical harmonics and compose like a representation; the edge frame puts
the edge on the polar (y) axis; the order-major layout and the inverse rescale have the documented shapes; the block as
a whole, and a model that uses it, are invariant / equivariant under global rotations and smooth across the blend of the
two frame quaternions."""
import math

import numpy as np
import pytest
import torch

from helpers import oracle_batch
from oracle import o3, tece
from tace_b200 import synth


def _random_rotation(seed):
    g = torch.Generator().manual_seed(seed)
    q, r = torch.linalg.qr(torch.randn(3, 3, generator=g, dtype=torch.float64))
    q = q * torch.sign(torch.diagonal(r))
    return q * torch.sign(torch.linalg.det(q))


def test_wigner_matrices_rotate_the_spherical_harmonics_and_compose():
    g = torch.Generator().manual_seed(0)
    v = torch.randn(7, 3, generator=g, dtype=torch.float64)
    v = v / v.norm(dim=1, keepdim=True)
    R1, R2 = _random_rotation(1), _random_rotation(2)
    for R in (R1, R2):
        blocks = tece.wigner_blocks(R[None], 3)
        Y, YR = o3.spherical_harmonics(3, v), o3.spherical_harmonics(3, v @ R.T)
        for l, D in enumerate(blocks):
            assert torch.allclose(YR[:, l * l:(l + 1) ** 2], Y[:, l * l:(l + 1) ** 2] @ D[0].T, atol=1e-12)
            assert torch.allclose(D[0] @ D[0].T, torch.eye(2 * l + 1, dtype=torch.float64), atol=1e-12)
    b1, b2, b12 = tece.wigner_blocks(R1[None], 3), tece.wigner_blocks(R2[None], 3), tece.wigner_blocks((R1 @ R2)[None], 3)
    for l in range(4):
        assert torch.allclose(b12[l][0], b1[l][0] @ b2[l][0], atol=1e-12)


def test_edge_frame_puts_the_edge_on_the_polar_axis():
    g = torch.Generator().manual_seed(3)
    v = torch.randn(200, 3, generator=g, dtype=torch.float64) * 2.0
    v[0] = torch.tensor([0.0, 1.0, 0.0]); v[1] = torch.tensor([0.0, -1.0, 0.0]); v[2] = torch.tensor([1e-9, -1.0, 0.0])
    R = tece.edge_rotation(v)
    assert torch.allclose(R @ R.transpose(1, 2), torch.eye(3, dtype=torch.float64).expand(200, 3, 3), atol=1e-6)
    assert torch.allclose(torch.linalg.det(R), torch.ones(200, dtype=torch.float64), atol=1e-6)
    u = v / v.norm(dim=1, keepdim=True)
    aligned = torch.einsum("eij,ej->ei", R, u)
    assert torch.allclose(aligned, torch.tensor([0.0, 1.0, 0.0], dtype=torch.float64).expand(200, 3), atol=1e-6)
    # in the edge frame only the m = 0 harmonics of the edge direction survive
    wig, wig_inv = tece.WignerD(2, 3).get_wigner(v)
    assert wig.shape == (200, 14, 16) and wig_inv.shape == (200, 16, 14)
    Y = o3.spherical_harmonics(3, u)
    rot = torch.einsum("emj,ej->em", wig, Y)
    assert torch.allclose(rot[:, 4:], torch.zeros(200, 10, dtype=torch.float64), atol=1e-5)
    assert torch.allclose(rot[:, :4], torch.tensor([math.sqrt(2 * l + 1) for l in range(4)], dtype=torch.float64).expand(200, 4), atol=1e-5)
    # inverse: transpose with l = 3 columns rescaled by sqrt(7 / 5)
    rows, ranks = tece.m_layout(3, 2)
    assert rows.tolist() == [0, 2, 6, 12, 3, 7, 13, 1, 5, 11, 8, 14, 4, 10]
    scale = torch.where(ranks > 2, math.sqrt(7.0 / 5.0), 1.0)
    assert torch.allclose(wig_inv, wig.transpose(1, 2) * scale, atol=1e-14)


def _conv(seed=0, C=8, heads=2):
    torch.manual_seed(seed)
    conv = tece.EdgeConvolution(2, 3, C, heads, 6, 8, 8, False, tece.ScaledSigmoid(), tece.ScaledSigmoid()).double()
    with torch.no_grad():  # zero in the reference's initialisation: make bias and phase matter
        conv.radial_proj.weight.normal_()
        conv.radial_proj.bias.normal_()
    return conv


def test_edge_block_is_equivariant_under_global_rotations():
    C = 8
    conv = _conv(C=C)
    g = torch.Generator().manual_seed(5)
    N, E = 6, 20
    x = torch.randn(N, 16, C, generator=g, dtype=torch.float64)
    ei = torch.stack([torch.randint(0, N, (E,), generator=g), torch.randint(0, N, (E,), generator=g)])
    vec = torch.randn(E, 3, generator=g, dtype=torch.float64)
    w = torch.randn(E, conv.weight_numel, generator=g, dtype=torch.float64)
    cutoff = torch.rand(E, 1, generator=g, dtype=torch.float64)
    radial = torch.randn(E, 8, generator=g, dtype=torch.float64)
    wd = tece.WignerD(2, 3)

    def run(x_, vec_):
        wig, wig_inv = wd.get_wigner(vec_)
        return conv(x_, w, ei, cutoff, wig, wig_inv, radial)

    out = run(x, vec)
    assert out.shape == (N, 16, 8)
    R = _random_rotation(7)
    D = torch.block_diag(*[b[0] for b in tece.wigner_blocks(R[None], 3)])
    out_rot = run(torch.einsum("ij,njc->nic", D, x), vec @ R.T)
    assert torch.allclose(out_rot, torch.einsum("ij,njc->nic", D, out), atol=1e-9)


def test_model_with_the_edge_block_is_invariant_and_smooth():
    """A two-layer model whose second interaction is the edge block: energy invariant under rotation, translation and
    atom permutation; forces rotate; finite differences of the energy match the autograd forces (which also run through
    the frame blend near the -y pole)."""
    from oracle.model import build_oracle

    s = synth.fcc_supercell(2, 3.61, 0.08, seed=4, species=(13, 29), fractions=(0.5, 0.5))
    cfg = synth.model_config(3, 8, 4.0, [13, 29], 12.0)
    cfg["atomic_basis"].update(type=["cgtp", "uv_so2"], num_head=2, edge_ace_hidden=4)
    cfg["mmax"] = 2
    torch.manual_seed(0)
    oracle = build_oracle(cfg, None, torch.float64)
    with torch.no_grad():
        for name, p in oracle.named_parameters():
            if "radial_proj" in name:
                p.normal_()
    data = oracle_batch([s], [13, 29], 4.0, torch.float64)
    ref = oracle(data)
    R = _random_rotation(9).numpy()
    s2 = dict(s, positions=s["positions"] @ R.T + 0.37, cell=s["cell"] @ R.T)
    ref2 = oracle(oracle_batch([s2], [13, 29], 4.0, torch.float64))
    assert abs(float(ref2["energy"][0] - ref["energy"][0])) < 1e-8
    assert np.abs(ref2["forces"].numpy() - ref["forces"].numpy() @ R.T).max() < 1e-7
    # finite differences
    h = 1e-5
    for atom, axis in ((0, 0), (3, 1), (5, 2)):
        e = []
        for sign in (+1, -1):
            p = s["positions"].copy()
            p[atom, axis] += sign * h
            e.append(float(oracle(oracle_batch([dict(s, positions=p)], [13, 29], 4.0, torch.float64))["energy"][0]))
        assert abs(-(e[0] - e[1]) / (2 * h) - float(ref["forces"][atom, axis])) < 1e-6


def test_full_order_wigner_rows_invert_exactly():
    """With every order kept (mmax == lmax) the inverse map undoes the rotation, as the reference's own round-trip test
    requires of WignerD(2, 2) (tests/test_o2.py:62-100); with mmax < lmax the product is the projector on the kept orders
    up to the sqrt((2l+1) / (2 mmax+1)) rescale of the higher ranks."""
    g = torch.Generator().manual_seed(11)
    v = torch.randn(7, 3, generator=g, dtype=torch.float64)
    wig, wig_inv = tece.WignerD(2, 2).get_wigner(v)
    assert wig.shape == (7, 9, 9)
    assert torch.allclose(torch.bmm(wig_inv, wig), torch.eye(9, dtype=torch.float64).expand(7, 9, 9), atol=1e-6)
    x = torch.randn(7, 9, generator=g, dtype=torch.float64)
    assert torch.allclose(torch.einsum("eij,ej->ei", wig_inv, torch.einsum("eij,ej->ei", wig, x)), x, atol=1e-6)
    wig, wig_inv = tece.WignerD(2, 3).get_wigner(v)
    prod = torch.bmm(wig, wig_inv)  # [14, 14]: rows of an orthogonal matrix times their rescaled transpose
    scale = torch.where(tece.m_layout(3, 2)[1] > 2, (7.0 / 5.0) ** 0.5, 1.0).to(torch.float64)
    assert torch.allclose(prod, torch.diag(scale).expand(7, 14, 14), atol=1e-6)
