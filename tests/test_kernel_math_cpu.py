"""The arithmetic headers the CUDA kernels are built from, compiled for the CPU and checked
against the oracle (values) and autograd (hand-written derivatives)."""
import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import o3
from oracle import model as om

DP = ctypes.POINTER(ctypes.c_double)


def ptr(a):
    return a.ctypes.data_as(DP)


def paths_and_layout(L, in1, outs):
    paths = [(l1, l2, l3) for l3 in outs for l1 in in1 for l2 in range(L + 1)
             if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0]
    k = {l: sum(1 for p in paths if p[2] == l) for l in outs}
    base, acc = {}, 0
    for l in outs:
        base[l] = acc
        acc += (2 * l + 1) * k[l]
    cnt = {l: 0 for l in outs}
    idx = []
    for (_, _, l3) in paths:
        idx.append([base[l3] + m3 * k[l3] + cnt[l3] for m3 in range(2 * l3 + 1)])
        cnt[l3] += 1
    return paths, idx, acc


def oracle_tp(L, Lin, x, Y, w):
    in1 = [0] if Lin < 0 else list(range(Lin + 1))
    irr1 = o3.Irreps([(1, l) for l in in1])
    irr2 = o3.Irreps.spherical_harmonics(L)
    paths, out = om.generate_paths(o3.Irreps([(1, l) for l in range(L + 1)]), irr1, irr2, "uvu")
    tp = om.TensorProduct(irr1, irr2, out, paths)
    return tp(x[None], Y[None], w[None])[0], out


RANK_PAIRS = [(L, Lx) for L in (1, 2, 3) for Lx in [-1] + list(range(1, L + 1))]  # (edge rank, source / output rank)


@pytest.mark.parametrize("L,Lin", RANK_PAIRS)
def test_interaction_tp_matches_oracle(cpu_harness, L, Lin):
    torch.manual_seed(L * 5 + Lin)
    scalar_src = Lin < 0
    dims = (ctypes.c_int * 4)()
    assert cpu_harness.h_tp_dims(L, Lin, dims) == 0
    NP, NX, NM, D = list(dims)
    in1 = [0] if scalar_src else list(range(Lin + 1))
    paths, idx, nm = paths_and_layout(L, in1, list(range(L + 1)))
    assert nm == NM and len(paths) == NP
    x = torch.randn(NX, dtype=torch.float64, requires_grad=True)
    Y = torch.randn(D, dtype=torch.float64, requires_grad=True)
    w = torch.randn(NP, dtype=torch.float64, requires_grad=True)
    ref, out_irreps = oracle_tp(L, Lin, x, Y, w)
    # oracle output: per path p a [1, 2l3+1] block, in path order
    perm = [i for blk in idx for i in blk]
    out = np.zeros(NM)
    z = np.zeros(max(NM, D, NX))
    xn, Yn, wn = x.detach().numpy(), Y.detach().numpy(), w.detach().numpy()
    cpu_harness.h_tp(L, Lin, 0, ptr(xn), ptr(Yn), ptr(wn), ptr(z), ptr(out), ptr(z), ptr(z))
    np.testing.assert_allclose(out[perm], ref.detach().numpy(), rtol=0, atol=1e-13)
    # backward against autograd
    g_ref = torch.randn(NM, dtype=torch.float64)  # gradient wrt oracle-ordered output
    dx_ref, dY_ref, dw_ref = torch.autograd.grad(ref, [x, Y, w], g_ref)
    g_mine = np.zeros(NM)
    g_mine[perm] = g_ref.numpy()
    dw, dY, dx = np.zeros(NP), np.zeros(D), np.zeros(NX)
    cpu_harness.h_tp(L, Lin, 1, ptr(xn), ptr(Yn), ptr(wn), ptr(g_mine), ptr(dw), ptr(dY), ptr(dx))
    np.testing.assert_allclose(dw, dw_ref.numpy(), rtol=0, atol=1e-12)
    np.testing.assert_allclose(dY, dY_ref.numpy(), rtol=0, atol=1e-12)
    if not scalar_src:  # the scalar-source layer never needs the source gradient
        np.testing.assert_allclose(dx, dx_ref.numpy(), rtol=0, atol=1e-12)


@pytest.mark.parametrize("L,Lin", RANK_PAIRS)
def test_backward_asks_for_weights_in_path_order(cpu_harness, L, Lin):
    """The kernels hand the generated backward code an accessor that produces a path's weight when it is asked for and
    consumes its gradient at once (one table entry in flight): every path must be asked for once, in ascending order,
    and its gradient handed back before the next weight is asked for.  The results equal those of the array form."""
    rng = np.random.default_rng(L * 7 + Lin)
    dims = (ctypes.c_int * 4)()
    assert cpu_harness.h_tp_dims(L, Lin, dims) == 0
    NP, NX, NM, D = list(dims)
    x, Y, w, g = rng.normal(size=NX), rng.normal(size=D), rng.normal(size=NP), rng.normal(size=NM)
    dw, dY, dx = np.zeros(NP), np.zeros(D), np.zeros(NX)
    cpu_harness.h_tp(L, Lin, 1, ptr(x), ptr(Y), ptr(w), ptr(g), ptr(dw), ptr(dY), ptr(dx))
    dw2, dY2, dx2 = np.zeros(NP), np.zeros(D), np.zeros(NX)
    assert cpu_harness.h_tp_bwd_ordered(L, Lin, ptr(x), ptr(Y), ptr(w), ptr(g), ptr(dw2), ptr(dY2), ptr(dx2)) == 0
    assert np.array_equal(dw, dw2) and np.array_equal(dY, dY2) and np.array_equal(dx, dx2)


@pytest.mark.parametrize("L,Lout", RANK_PAIRS)
def test_product_basis_matches_oracle(cpu_harness, L, Lout):
    torch.manual_seed(10 + L)
    D = (L + 1) ** 2
    outs = [0] if Lout < 0 else list(range(Lout + 1))
    irr = o3.Irreps([(1, l) for l in range(L + 1)])
    paths, out = om.generate_paths(o3.Irreps([(1, l) for l in outs]), irr, irr, "uuu", identical_inputs=True)
    tp = om.TensorProduct(irr, irr, out, paths)
    a = torch.randn(D, dtype=torch.float64, requires_grad=True)
    ref = tp(a[None], a[None])[0]
    _, idx, nb = paths_and_layout(L, list(range(L + 1)), outs)
    perm = [i for blk in idx for i in blk]
    b = np.zeros(nb)
    assert cpu_harness.h_pb(L, Lout, 0, ptr(a.detach().numpy()), ptr(b), ptr(b)) == nb
    np.testing.assert_allclose(b[perm], ref.detach().numpy(), rtol=0, atol=1e-13)
    g_ref = torch.randn(nb, dtype=torch.float64)
    (da_ref,) = torch.autograd.grad(ref, [a], g_ref)
    g_mine = np.zeros(nb)
    g_mine[perm] = g_ref.numpy()
    da = np.zeros(D)
    cpu_harness.h_pb(L, Lout, 1, ptr(a.detach().numpy()), ptr(g_mine), ptr(da))
    np.testing.assert_allclose(da, da_ref.numpy(), rtol=0, atol=1e-12)


@pytest.mark.parametrize("L,Lout", RANK_PAIRS)
def test_third_order_product_basis_matches_oracle(cpu_harness, L, Lout):
    """(A x A) x A of correlation 3: values against the oracle's tensor product, both gradients against autograd."""
    torch.manual_seed(20 + L)
    D = (L + 1) ** 2
    ls = list(range(L + 1))
    outs = [0] if Lout < 0 else list(range(Lout + 1))
    irr = o3.Irreps([(1, l) for l in ls])
    paths2, out2 = om.generate_paths(irr, irr, irr, "uuu", identical_inputs=True)       # every rank keeps its slots
    paths3, out3 = om.generate_paths(o3.Irreps([(1, l) for l in outs]), out2, irr, "uuu")
    tp3 = om.TensorProduct(out2, irr, out3, paths3)
    _, idx2, nb2 = paths_and_layout(L, ls, ls)
    perm2 = [i for blk in idx2 for i in blk]                                            # oracle order -> slot layout
    # layout of the third-order output: [l3][m3][path], paths in oracle order
    l3_of = [l for _, l in out3]
    k = {l: l3_of.count(l) for l in outs}
    base, acc = {}, 0
    for l in outs:
        base[l] = acc
        acc += (2 * l + 1) * k[l]
    cnt, perm3 = {l: 0 for l in outs}, []
    for l in l3_of:
        perm3 += [base[l] + m * k[l] + cnt[l] for m in range(2 * l + 1)]
        cnt[l] += 1
    a = torch.randn(D, dtype=torch.float64, requires_grad=True)
    b2_oracle = torch.randn(nb2, dtype=torch.float64, requires_grad=True)
    ref = tp3(b2_oracle[None], a[None])[0]
    b2_mine = np.zeros(nb2)
    b2_mine[perm2] = b2_oracle.detach().numpy()
    b3 = np.zeros(acc)
    z = np.zeros(max(acc, nb2, D))
    assert cpu_harness.h_pb3(L, Lout, 0, ptr(a.detach().numpy()), ptr(b2_mine), ptr(z), ptr(b3), ptr(z)) == acc
    np.testing.assert_allclose(b3[perm3], ref.detach().numpy(), rtol=0, atol=1e-13)
    g_ref = torch.randn(acc, dtype=torch.float64)
    db2_ref, da_ref = torch.autograd.grad(ref, [b2_oracle, a], g_ref)
    g_mine = np.zeros(acc)
    g_mine[perm3] = g_ref.numpy()
    db2, da = np.zeros(nb2), np.zeros(D)
    cpu_harness.h_pb3(L, Lout, 1, ptr(a.detach().numpy()), ptr(b2_mine), ptr(g_mine), ptr(db2), ptr(da))
    np.testing.assert_allclose(db2[perm2], db2_ref.numpy(), rtol=0, atol=1e-12)
    np.testing.assert_allclose(da, da_ref.numpy(), rtol=0, atol=1e-12)


def test_radial_basis_without_envelope_and_the_envelope_itself(cpu_harness):
    """radial_basis.apply_cutoff = False: plain Bessel features plus the envelope (value, derivative) on its own."""
    torch.set_default_dtype(torch.float64)
    try:
        rb = om.RadialBasis(5.0, 8, 5, apply_cutoff=False)
    finally:
        torch.set_default_dtype(torch.float32)
    cpu_harness.h_radial2.argtypes = [ctypes.c_double, ctypes.c_double, ctypes.c_int, ctypes.c_int, DP, DP, DP]
    for d0 in [0.8, 2.553, 4.2, 4.999, 5.3]:
        d = torch.tensor([[d0]], dtype=torch.float64, requires_grad=True)
        feats, env = rb(d)
        jac = torch.stack([torch.autograd.grad(feats[0, i], d, retain_graph=True)[0][0, 0] for i in range(8)])
        (denv,) = torch.autograd.grad(env[0, 0], d, allow_unused=True)
        b, db, e = np.zeros(8), np.zeros(8), np.zeros(2)
        cpu_harness.h_radial2(d0, 5.0, 5, 1, ptr(b), ptr(db), ptr(e))
        np.testing.assert_allclose(b, feats[0].detach().numpy(), rtol=0, atol=1e-13)
        np.testing.assert_allclose(db, jac.numpy(), rtol=0, atol=1e-12)
        assert abs(e[0] - env.item()) < 1e-14 and abs(e[1] - (0.0 if denv is None else denv.item())) < 1e-12


@pytest.mark.parametrize("L", [1, 2, 3])
def test_spherical_harmonics_and_gradient(cpu_harness, L):
    torch.manual_seed(L)
    D = (L + 1) ** 2
    n = torch.randn(3, dtype=torch.float64) * 0.7
    n.requires_grad_(True)
    ref = o3.spherical_harmonics(L, n[None], "component")[0]
    Y = np.zeros(D)
    cpu_harness.h_sh(L, ptr(n.detach().numpy()), ptr(Y))
    np.testing.assert_allclose(Y, ref.detach().numpy(), rtol=0, atol=1e-13)
    dY = torch.randn(D, dtype=torch.float64)
    (dn_ref,) = torch.autograd.grad(ref, [n], dY)
    dn = np.zeros(3)
    cpu_harness.h_sh_grad(L, ptr(n.detach().numpy()), ptr(dY.numpy()), ptr(dn))
    np.testing.assert_allclose(dn, dn_ref.numpy(), rtol=0, atol=1e-12)


def test_radial_basis_and_gradient(cpu_harness):
    torch.set_default_dtype(torch.float64)
    try:
        rb = om.RadialBasis(5.0, 8, 5)
    finally:
        torch.set_default_dtype(torch.float32)
    for d0 in [0.8, 2.553, 4.2, 4.999, 5.0, 5.3]:
        d = torch.tensor([[d0]], dtype=torch.float64, requires_grad=True)
        ref = rb(d)[0][0]
        jac = torch.stack([torch.autograd.grad(ref[i], d, retain_graph=True)[0][0, 0] for i in range(8)])
        b, db = np.zeros(8), np.zeros(8)
        cpu_harness.h_radial.argtypes = [ctypes.c_double, ctypes.c_double, ctypes.c_int, DP, DP]
        cpu_harness.h_radial(d0, 5.0, 5, ptr(b), ptr(db))
        np.testing.assert_allclose(b, ref.detach().numpy(), rtol=0, atol=1e-13)
        np.testing.assert_allclose(db, jac.numpy(), rtol=0, atol=1e-12)


def test_radial_mlp_hidden_layers(cpu_harness):
    torch.manual_seed(3)
    mlp = om.MLP([8, 64, 64, 64, 11]).double()
    lins = [m for m in mlp.mlp if isinstance(m, om.MlpLinear)]
    A = [(l.weight * l.alpha).detach().numpy().copy() for l in lins[:3]]
    At = [np.ascontiguousarray(a.T) for a in A]
    b = torch.randn(1, 8, dtype=torch.float64, requires_grad=True)
    h3_ref = torch.nn.functional.silu(mlp.mlp[4](mlp.mlp[3](mlp.mlp[2](mlp.mlp[1](mlp.mlp[0](b))))))
    dh3 = torch.randn(1, 64, dtype=torch.float64)
    (db_ref,) = torch.autograd.grad(h3_ref, [b], dh3)
    h3, db = np.zeros(64), np.zeros(8)
    cpu_harness.h_mlp(ptr(b.detach().numpy()), ptr(A[0]), ptr(A[1]), ptr(A[2]), ptr(At[1]), ptr(At[2]),
                      ptr(dh3.numpy()), ptr(h3), ptr(db))
    np.testing.assert_allclose(h3, h3_ref.detach().numpy()[0], rtol=0, atol=1e-13)
    np.testing.assert_allclose(db, db_ref.numpy()[0], rtol=0, atol=1e-12)


def test_edge_vector_gradient(cpu_harness):
    torch.manual_seed(5)
    v = torch.randn(3, dtype=torch.float64, requires_grad=True)
    d = (v**2).sum().sqrt() + 1e-9
    n = v / d
    dd, dn = torch.randn((), dtype=torch.float64), torch.randn(3, dtype=torch.float64)
    (g_ref,) = torch.autograd.grad(d * dd + (n * dn).sum(), [v])
    g = np.zeros(3)
    cpu_harness.h_edge_grad.argtypes = [DP, ctypes.c_double, DP, DP]
    cpu_harness.h_edge_grad(ptr(v.detach().numpy()), float(dd), ptr(dn.numpy()), ptr(g))
    np.testing.assert_allclose(g, g_ref.numpy(), rtol=0, atol=1e-12)


def test_generated_header_is_what_its_generator_writes():
    """``tp_gen.cuh`` is committed so that a build needs no generator run; it must not drift from ``gen_tables.py``."""
    import importlib.util
    import os

    csrc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tace_b200", "csrc")
    spec = importlib.util.spec_from_file_location("tace_gen_tables", os.path.join(csrc, "gen_tables.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    text, summary = gen.generate()
    with open(os.path.join(csrc, "tp_gen.cuh")) as fh:
        assert fh.read() == text
    assert any(s["tag"] == "L3_F" and s["P"] == 23 and s["nm"] == 99 for s in summary)
