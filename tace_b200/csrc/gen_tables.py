#!/usr/bin/env python
"""Generates ``tp_gen.cuh``: path tables and straight-line contraction code.

Run ``python tace_b200/csrc/gen_tables.py`` after changing the path rules; the
generated header is committed.  The coupling coefficients are the real-basis
Wigner-3j symbols (SU(2) Clebsch-Gordan coefficients conjugated into the real
spherical-harmonic basis with polar axis y, unit Frobenius norm) times
sqrt(2 l3 + 1), which is what the reference's e3nn ``TensorProduct`` applies
per path (``tace/models/_e3nn/fused.py:44-51,203-210``); path order follows
``tace/models/_e3nn/paths.py:30-71`` (output rank major, then first input,
then second input).

Everything emitted is plain C++ (``TACE_HD`` = ``__host__ __device__``), so the
same code is exercised on the CPU by the unit tests and on the GPU by the
kernels.
"""

from __future__ import annotations

import math
import os
from math import factorial as f

import numpy as np


# ---------------------------------------------------------------------------- 3j
def _cg(j1, m1, j2, m2, j3, m3):
    """<j1 m1 j2 m2|j3 m3> by the standard (Condon-Shortley) sum over k."""
    if m1 + m2 != m3:
        return 0.0
    pref = math.sqrt((2 * j3 + 1) * f(j3 + j1 - j2) * f(j3 - j1 + j2) * f(j1 + j2 - j3) / f(j1 + j2 + j3 + 1))
    pref *= math.sqrt(f(j3 + m3) * f(j3 - m3) * f(j1 - m1) * f(j1 + m1) * f(j2 - m2) * f(j2 + m2))
    s = 0.0
    for k in range(0, j1 + j2 - j3 + 1):
        args = [k, j1 + j2 - j3 - k, j1 - m1 - k, j2 + m2 - k, j3 - j2 + m1 + k, j3 - j1 - m2 + k]
        if min(args) < 0:
            continue
        d = 1.0
        for a in args:
            d *= f(a)
        s += (-1) ** k / d
    return pref * s


def _q(l):
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    for m in range(-l, 0):
        q[l + m, l + abs(m)] = 1 / math.sqrt(2)
        q[l + m, l - abs(m)] = -1j / math.sqrt(2)
    q[l, l] = 1
    for m in range(1, l + 1):
        q[l + m, l + abs(m)] = (-1) ** m / math.sqrt(2)
        q[l + m, l - abs(m)] = 1j * (-1) ** m / math.sqrt(2)
    return (-1j) ** l * q


_W3J = {}


def w3j(l1, l2, l3):
    key = (l1, l2, l3)
    if key not in _W3J:
        c = np.zeros((2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1), dtype=np.complex128)
        for m1 in range(-l1, l1 + 1):
            for m2 in range(-l2, l2 + 1):
                if abs(m1 + m2) <= l3:
                    c[l1 + m1, l2 + m2, l3 + m1 + m2] = _cg(l1, m1, l2, m2, l3, m1 + m2)
        c = np.einsum("ij,kl,mn,ikn->jlm", _q(l1), _q(l2), np.conj(_q(l3).T), c)
        assert np.abs(c.imag).max() < 1e-12
        c = c.real
        c[np.abs(c) < 1e-14] = 0.0
        _W3J[key] = c / np.linalg.norm(c)
    return _W3J[key]


# ------------------------------------------------------------------------- paths
def tp_paths(L, in1_ls, in2_ls, out_ls):
    paths = []
    for l3 in out_ls:
        for l1 in in1_ls:
            for l2 in in2_ls:
                if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0:
                    paths.append((l1, l2, l3))
    return paths


class Layout:
    """Message layout [l3][m3][p_local]: index = base[l3] + m3 * k[l3] + p_local."""

    def __init__(self, paths, out_ls):
        self.paths = paths
        self.k = {l: sum(1 for p in paths if p[2] == l) for l in out_ls}
        self.base, acc = {}, 0
        for l in out_ls:
            self.base[l] = acc
            acc += (2 * l + 1) * self.k[l]
        self.nm = acc
        self.plocal, cnt = [], {l: 0 for l in out_ls}
        for (_, _, l3) in paths:
            self.plocal.append(cnt[l3])
            cnt[l3] += 1

    def idx(self, p, m3):
        l3 = self.paths[p][2]
        return self.base[l3] + m3 * self.k[l3] + self.plocal[p]


def lit(v):
    return f"T({v!r})"


# ----------------------------------------------------------- interaction TP code
def gen_interaction(L, Lin, out):
    """Emits, for edge / message rank L (angular features and messages carry ranks 0..L) and source rank Lin
    (source features carry ranks 0..Lin; Lin < 0: scalar source, the first layer):

    * ``build_G``: the channel-independent coupling of one edge, G[i] = sum_m2 K^p[m1,m2,m3] Y[l2,m2]
      for every structurally non-zero (p, m1, m3), ordered output-group major, then (p, m3, m1), each
      group padded to a multiple of four entries so the kernels read it with 128-bit loads;
    * ``fwd<g>``: message components of output group g (ranks are split into at most two groups to
      halve the accumulator registers per thread);
    * ``bwd``: gradients with respect to the per-edge weights, the angular features and the source
      features of one (edge, channel).
    """
    scalar_src = Lin < 0
    tag = f"L{L}_" + ("S" if scalar_src else "F" if Lin == L else f"N{Lin}")
    in1 = [0] if scalar_src else list(range(Lin + 1))
    sh = list(range(L + 1))
    outs = list(range(L + 1))
    paths = tp_paths(L, in1, sh, outs)
    lay = Layout(paths, outs)
    xoff = {l: (0 if scalar_src else l * l) for l in in1}
    nx = 1 if scalar_src else (Lin + 1) ** 2
    D = (L + 1) ** 2
    P = len(paths)
    Ks = [w3j(*p) * math.sqrt(2 * p[2] + 1) for p in paths]
    nnz_l3 = {l: sum(int(np.count_nonzero(K)) for K, p in zip(Ks, paths) if p[2] == l) for l in outs}
    # output-rank groups: one group for small cases, otherwise split at the rank that balances the work
    if scalar_src or L < 3:  # up to rank 2 one thread holds every message component of a channel (35 accumulators)
        groups = [outs]
    else:
        best = min(range(1, L + 1), key=lambda c: abs(sum(nnz_l3[l] for l in outs[:c]) - sum(nnz_l3[l] for l in outs[c:])))
        groups = [outs[:best], outs[best:]]
    gi, terms = {}, []          # compact index of (p, m1, m3); per entry the list of (y index, coefficient)
    grp_goff, grp_gcnt, grp_p0, grp_np, grp_m0, grp_nm = [], [], [], [], [], []
    for ls in groups:
        while len(terms) % 4:
            terms.append([])     # padding entry (stays zero)
        grp_goff.append(len(terms))
        ps = [p for p, pt in enumerate(paths) if pt[2] in ls]
        grp_p0.append(ps[0]); grp_np.append(len(ps))
        grp_m0.append(lay.base[ls[0]]); grp_nm.append(sum((2 * l + 1) * lay.k[l] for l in ls))
        for p in ps:
            l1, l2, l3 = paths[p]
            K = Ks[p]
            for m3 in range(2 * l3 + 1):
                for m1 in range(2 * l1 + 1):
                    t = [(l2 * l2 + m2, K[m1, m2, m3]) for m2 in range(2 * l2 + 1) if K[m1, m2, m3] != 0.0]
                    if t:
                        gi[(p, m1, m3)] = len(terms)
                        terms.append(t)
        grp_gcnt.append(len(terms) - grp_goff[-1])
    while len(terms) % 4:
        terms.append([])
    ng = len(terms)
    nnz_total = sum(int(np.count_nonzero(K)) for K in Ks)
    ngrp = len(groups)

    o = out.append
    o(f"// ---- interaction tensor product, L={L}, {'scalar' if scalar_src else f'rank <= {Lin}'} source: {P} paths, "
      f"{lay.nm} message components, {len(gi)} non-zero G entries (padded to {ng}), {nnz_total} coupling non-zeros, "
      f"output groups {groups}")
    o(f"static const int tp_{tag}_k[{L + 1}] = {{{', '.join(str(lay.k[l]) for l in outs)}}};")
    o(f"static const int tp_{tag}_base[{L + 1}] = {{{', '.join(str(lay.base[l]) for l in outs)}}};")
    o(f"struct TPX_{tag} {{")
    o(f"  static constexpr int L = {L}, NP = {P}, NX = {nx}, NM = {lay.nm}, NG = {ng}, D = {D}, NGRP = {ngrp};")
    for name, arr in [("GOFF", grp_goff), ("GCNT", [((c + 3) // 4) * 4 for c in grp_gcnt]), ("P0", grp_p0), ("NPG", grp_np),
                      ("M0", grp_m0), ("NMG", grp_nm)]:
        o(f"  static constexpr int {name}0 = {arr[0]}, {name}1 = {arr[-1]};")
    # build_G in parts: each output group's entries are cut into two halves so that four threads (two per
    # group) can build one edge's row cooperatively inside the tensor-product kernels
    part_bounds = []
    for g in range(ngrp):
        lo, hi = grp_goff[g], grp_goff[g] + ((grp_gcnt[g] + 3) // 4) * 4
        mid = lo + (((hi - lo) // 2 + 3) // 4) * 4
        part_bounds += [(lo, mid), (mid, hi)]
    o(f"  static constexpr int NPART = {len(part_bounds)};")
    o(f"  template <int PART, typename T> static TACE_HD TACE_INLINE void build_G_part(const T* __restrict__ Y, T* __restrict__ G) {{")
    for pi, (lo, hi) in enumerate(part_bounds):
        o(f"    if constexpr (PART == {pi}) {{")
        for i in range(lo, hi):
            t = terms[i]
            expr = " + ".join(f"{lit(float(c))} * Y[{y}]" for y, c in t) if t else "T(0)"
            o(f"      G[{i}] = {expr};")
        o("    }")
    o("  }")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void build_G(const T (&Y)[{D}], T* __restrict__ G) {{")
    for pi in range(len(part_bounds)):
        o(f"    build_G_part<{pi}, T>(Y, G);")
    o("  }")

    def load_G(lo, hi, loaded):
        """Emit 4-wide loads covering entries [lo, hi); returns the lines."""
        lines = []
        for j in range(lo // 4, (hi + 3) // 4):
            if j not in loaded:
                loaded.add(j)
                lines.append(f"    T G_{4 * j}, G_{4 * j + 1}, G_{4 * j + 2}, G_{4 * j + 3}; "
                             f"ld4(G + {4 * j}, G_{4 * j}, G_{4 * j + 1}, G_{4 * j + 2}, G_{4 * j + 3});")
        return lines

    # forward per group: acc[local idx] += w[p_local] * sum_m1 x[m1] G[m1][m3]; G points at the edge's full row
    for g, ls in enumerate(groups):
        ps = [p for p, pt in enumerate(paths) if pt[2] in ls]
        o(f"  template <typename T> static TACE_HD TACE_INLINE void fwd{g}(const T (&x)[{nx}], const T* __restrict__ G, "
          f"const T (&w)[{grp_np[g]}], T (&acc)[{grp_nm[g]}]) {{")
        loaded = set()
        for p in ps:
            l1, l2, l3 = paths[p]
            ids = [gi[(p, m1, m3)] for m3 in range(2 * l3 + 1) for m1 in range(2 * l1 + 1) if (p, m1, m3) in gi]
            for line in load_G(min(ids), max(ids) + 1, loaded):
                o(line)
            for m3 in range(2 * l3 + 1):
                ts = [f"x[{xoff[l1] + m1}] * G_{gi[(p, m1, m3)]}" for m1 in range(2 * l1 + 1) if (p, m1, m3) in gi]
                if ts:
                    o(f"    acc[{lay.idx(p, m3) - grp_m0[g]}] += w[{p - grp_p0[g]}] * ({' + '.join(ts)});")
        o("  }")

    if ngrp == 1:  # single group: fwd1 is never launched, but must exist for the kernel template
        o(f"  template <typename T> static TACE_HD TACE_INLINE void fwd1(const T (&x)[{nx}], const T* __restrict__ G, "
          f"const T (&w)[{grp_np[0]}], T (&acc)[{grp_nm[0]}]) {{ fwd0<T>(x, G, w, acc); }}")

    # backward of one (edge, channel): g is read from gs[k * gstride] (the target's message gradient, channel c).  The
    # path weights come from, and their gradients go to, an accessor: wf.get<p>() is called once when the block of path p
    # starts (paths in ascending order) and wf.put<p>(dE/dw_p) once when it ends, so a caller may produce a weight just
    # before it is needed and consume its gradient at once instead of holding all of them in registers.
    o(f"  template <typename T> static TACE_HD TACE_INLINE void bwd(const T (&x)[{nx}], const T* __restrict__ gs, int gstride, "
      f"const T* __restrict__ G, const T (&w)[{P}], T (&dw)[{P}], T (&dY)[{D}], T (&dx)[{nx}]) {{")
    o(f"    TpArrayWeights<T> wf{{w, dw}};")
    o(f"    bwd_w<T>(x, gs, gstride, G, wf, dY, dx);")
    o("  }")
    o(f"  template <typename T, typename WF> static TACE_HD TACE_INLINE void bwd_w(const T (&x)[{nx}], const T* __restrict__ gs, "
      f"int gstride, const T* __restrict__ G, WF& wf, T (&dY)[{D}], T (&dx)[{nx}]) {{")
    for p, (l1, l2, l3) in enumerate(paths):
        K = Ks[p]
        n3 = 2 * l3 + 1
        pairs = [(m1, m3) for m3 in range(n3) for m1 in range(2 * l1 + 1) if (p, m1, m3) in gi]
        ids = [gi[(p, m1, m3)] for m1, m3 in pairs]
        o("  {")
        o(f"    const T w{p} = wf.template get<{p}>();")
        for line in load_G(min(ids), max(ids) + 1, set()):
            o(line)
        for m3 in range(n3):
            o(f"    const T g{m3} = gs[{lay.idx(p, m3)} * gstride];")
        # u[m1] = sum_m3 G[m1][m3] g[m3] serves both the weight gradient (dw = sum_m1 x[m1] u[m1]) and the source
        # gradient (dx[m1] += w u[m1]); the outer products q = x (x) g are only needed for the angular gradient
        us = []
        for m1 in range(2 * l1 + 1):
            ts = [f"G_{gi[(p, m1, m3)]} * g{m3}" for m3 in range(n3) if (p, m1, m3) in gi]
            if ts:
                o(f"    const T u{m1} = {' + '.join(ts)};")
                us.append(m1)
        o(f"    wf.template put<{p}>({' + '.join(f'x[{xoff[l1] + m1}] * u{m1}' for m1 in us)});")
        if not scalar_src:
            for m1 in us:
                o(f"    dx[{xoff[l1] + m1}] += w{p} * u{m1};")
        used = sorted({(m1, m3) for m1, m3 in pairs if any(K[m1, m2, m3] != 0.0 for m2 in range(2 * l2 + 1))})
        for m1, m3 in used:
            o(f"    const T q{m1}_{m3} = x[{xoff[l1] + m1}] * g{m3};")
        for m2 in range(2 * l2 + 1):
            ts = [f"{lit(float(K[m1, m2, m3]))} * q{m1}_{m3}" for m1, m3 in pairs if K[m1, m2, m3] != 0.0]
            if ts:
                o(f"    dY[{l2 * l2 + m2}] += w{p} * ({' + '.join(ts)});")
        o("  }")
    o("  }")
    o("};")
    return dict(tag=tag, P=P, nm=lay.nm, ng=ng, nnz=nnz_total, groups=groups, gcnt=grp_gcnt, nmg=grp_nm)


# ------------------------------------------------------------- product basis code
def gen_product(L, Lout, out):
    """Input ranks 0..L, output ranks 0..Lout (Lout < 0: scalar outputs only, the last layer)."""
    last = Lout < 0
    tag = f"L{L}_" + ("T" if last else "A" if Lout == L else f"N{Lout}")  # T = target (scalar) outputs, A = all ranks
    ls = list(range(L + 1))
    outs = [0] if last else list(range(Lout + 1))
    paths = tp_paths(L, ls, ls, outs)
    lay = Layout(paths, outs)
    D = (L + 1) ** 2
    P = len(paths)
    o = out.append
    nnz = sum(int(np.count_nonzero(w3j(*p))) for p in paths)
    o(f"// ---- product basis (A x A), L={L}, {'scalar outputs' if last else f'output ranks <= {Lout}'}: {P} paths, "
      f"{lay.nm} components, {nnz} coupling non-zeros")
    o(f"struct PB_{tag} {{ static constexpr int L = {L}, NP = {P}, NB = {lay.nm}, D = {D}; }};")
    o(f"static const int pb_{tag}_k[{len(outs)}] = {{{', '.join(str(lay.k[l]) for l in outs)}}};")
    o(f"static const int pb_{tag}_base[{len(outs)}] = {{{', '.join(str(lay.base[l]) for l in outs)}}};")
    o("template <typename T>")
    o(f"TACE_HD TACE_INLINE void pb_fwd_{tag}(const T (&a)[{D}], T (&b)[{lay.nm}]) {{")
    for p, (l1, l2, l3) in enumerate(paths):
        K = w3j(l1, l2, l3) * math.sqrt(2 * l3 + 1)
        for m3 in range(2 * l3 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * a[{l1 * l1 + m1}] * a[{l2 * l2 + m2}]"
                     for m1 in range(2 * l1 + 1) for m2 in range(2 * l2 + 1) if K[m1, m2, m3] != 0.0]
            o(f"  b[{lay.idx(p, m3)}] = {' + '.join(terms) if terms else 'T(0)'};")
    o("}")
    o("template <typename T>")
    o(f"TACE_HD TACE_INLINE void pb_bwd_{tag}(const T (&a)[{D}], const T (&db)[{lay.nm}], T (&da)[{D}]) {{")
    for p, (l1, l2, l3) in enumerate(paths):
        K = w3j(l1, l2, l3) * math.sqrt(2 * l3 + 1)
        for m1 in range(2 * l1 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * a[{l2 * l2 + m2}] * db[{lay.idx(p, m3)}]"
                     for m2 in range(2 * l2 + 1) for m3 in range(2 * l3 + 1) if K[m1, m2, m3] != 0.0]
            if terms:
                o(f"  da[{l1 * l1 + m1}] += {' + '.join(terms)};")
        for m2 in range(2 * l2 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * a[{l1 * l1 + m1}] * db[{lay.idx(p, m3)}]"
                     for m1 in range(2 * l1 + 1) for m3 in range(2 * l3 + 1) if K[m1, m2, m3] != 0.0]
            if terms:
                o(f"  da[{l2 * l2 + m2}] += {' + '.join(terms)};")
    o("}")
    o(f"struct PBX_{tag} : PB_{tag} {{")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void fwd(const T (&a)[{D}], T (&b)[{lay.nm}]) {{ pb_fwd_{tag}<T>(a, b); }}")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void bwd(const T (&a)[{D}], const T (&db)[{lay.nm}], T (&da)[{D}]) "
      f"{{ pb_bwd_{tag}<T>(a, db, da); }}")
    o("};")
    return dict(tag=tag, P=P, nb=lay.nm, nnz=nnz)


def bilinear_paths(L, outs):
    """Paths of the gated bilinear product (tace/models/_e3nn/prod.py:87-111, paths.py:30-71): first factor ranks 0..L,
    second factor ranks 0..L followed by a block of ones (rank 0, written l2 = -1 here), output-rank major."""
    paths = []
    for l3 in outs:
        for l1 in range(L + 1):
            for l2 in range(L + 1):
                if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0:
                    paths.append((l1, l2, l3))
            if l1 == l3:
                paths.append((l1, -1, l3))
    return paths


def gen_product_bilinear(L, Lout, out):
    """b[p, m3] = w[p] * sum K x[l1, m1] y[l2, m2] for two different factors and one weight per path; the paths whose
    second factor is the block of ones reduce to w[p] * x[l3, m3].  Backward: dx, dy (accumulated) and dw."""
    last = Lout < 0
    tag = f"L{L}_" + ("T" if last else "A" if Lout == L else f"N{Lout}")
    outs = [0] if last else list(range(Lout + 1))
    paths = bilinear_paths(L, outs)
    lay = Layout(paths, outs)
    D = (L + 1) ** 2
    P = len(paths)
    o = out.append
    o(f"// ---- gated bilinear product (x (x) [y, 1]), L={L}, {'scalar outputs' if last else f'output ranks <= {Lout}'}: {P} paths, "
      f"{lay.nm} components")
    o(f"struct PBL_{tag} {{ static constexpr int L = {L}, NP = {P}, NB = {lay.nm}, D = {D}; }};")
    o(f"static const int pbl_{tag}_k[{len(outs)}] = {{{', '.join(str(lay.k[l]) for l in outs)}}};")
    o(f"static const int pbl_{tag}_base[{len(outs)}] = {{{', '.join(str(lay.base[l]) for l in outs)}}};")

    def coupling(l1, l2, l3):
        return w3j(l1, l2, l3) * math.sqrt(2 * l3 + 1)

    o(f"struct PBLX_{tag} : PBL_{tag} {{")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void fwd(const T (&x)[{D}], const T (&y)[{D}], const T (&w)[{P}], T (&b)[{lay.nm}]) {{")
    for p, (l1, l2, l3) in enumerate(paths):
        for m3 in range(2 * l3 + 1):
            if l2 < 0:
                o(f"    b[{lay.idx(p, m3)}] = w[{p}] * x[{l1 * l1 + m3}];")
                continue
            K = coupling(l1, l2, l3)
            terms = [f"{lit(float(K[m1, m2, m3]))} * x[{l1 * l1 + m1}] * y[{l2 * l2 + m2}]"
                     for m1 in range(2 * l1 + 1) for m2 in range(2 * l2 + 1) if K[m1, m2, m3] != 0.0]
            o(f"    b[{lay.idx(p, m3)}] = w[{p}] * ({' + '.join(terms) if terms else 'T(0)'});")
    o("  }")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void bwd(const T (&x)[{D}], const T (&y)[{D}], const T (&w)[{P}], "
      f"const T (&db)[{lay.nm}], T (&dx)[{D}], T (&dy)[{D}], T (&dw)[{P}]) {{")
    for p, (l1, l2, l3) in enumerate(paths):
        if l2 < 0:
            terms = [f"x[{l1 * l1 + m}] * db[{lay.idx(p, m)}]" for m in range(2 * l3 + 1)]
            o(f"    dw[{p}] = {' + '.join(terms)};")
            for m in range(2 * l3 + 1):
                o(f"    dx[{l1 * l1 + m}] += w[{p}] * db[{lay.idx(p, m)}];")
            continue
        K = coupling(l1, l2, l3)
        o("    {")
        o(f"      T s = T(0), t;")
        for m3 in range(2 * l3 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * x[{l1 * l1 + m1}] * y[{l2 * l2 + m2}]"
                     for m1 in range(2 * l1 + 1) for m2 in range(2 * l2 + 1) if K[m1, m2, m3] != 0.0]
            if terms:
                o(f"      s += db[{lay.idx(p, m3)}] * ({' + '.join(terms)});")
        o(f"      dw[{p}] = s;")
        for m1 in range(2 * l1 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * y[{l2 * l2 + m2}] * db[{lay.idx(p, m3)}]"
                     for m2 in range(2 * l2 + 1) for m3 in range(2 * l3 + 1) if K[m1, m2, m3] != 0.0]
            if terms:
                o(f"      t = {' + '.join(terms)}; dx[{l1 * l1 + m1}] += w[{p}] * t;")
        for m2 in range(2 * l2 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * x[{l1 * l1 + m1}] * db[{lay.idx(p, m3)}]"
                     for m1 in range(2 * l1 + 1) for m3 in range(2 * l3 + 1) if K[m1, m2, m3] != 0.0]
            if terms:
                o(f"      t = {' + '.join(terms)}; dy[{l2 * l2 + m2}] += w[{p}] * t;")
        o("    }")
    o("  }")
    o("};")
    return dict(tag="bilinear " + tag, P=P, nb=lay.nm)


def gen_product3(L, Lout, out):
    """Third-order product basis B3 = (A x A) x A (correlation 3, tace/models/_e3nn/prod.py:216-266): the first factor
    is the full second-order basis (every path of ranks <= L keeps its own slot, layout of PB_L{L}_A), the second is A,
    outputs carry ranks 0..Lout (Lout < 0: scalars only).  B3 (593 components at L = 3) does not fit in registers, so
    the forward code stores each component through a strided pointer and the backward pass comes as two functions,
    one per operand, that read the gradient of B3 the same way."""
    last = Lout < 0
    tag = f"L{L}_" + ("T" if last else "A" if Lout == L else f"N{Lout}")
    ls = list(range(L + 1))
    outs = [0] if last else list(range(Lout + 1))
    slots = tp_paths(L, ls, ls, ls)                 # second-order paths = slots of the first operand
    lay2 = Layout(slots, ls)
    paths = [(s, lb, l3) for l3 in outs for s, (_, _, lsl) in enumerate(slots) for lb in ls
             if abs(lsl - lb) <= l3 <= lsl + lb and (lsl + lb + l3) % 2 == 0]
    lay3 = Layout([(slots[s][2], lb, l3) for s, lb, l3 in paths], outs)
    D = (L + 1) ** 2
    o = out.append
    nnz = sum(int(np.count_nonzero(w3j(slots[s][2], lb, l3))) for s, lb, l3 in paths)
    o(f"// ---- third-order product basis ((A x A) x A), L={L}, {'scalar outputs' if last else f'output ranks <= {Lout}'}: "
      f"{len(paths)} paths, {lay3.nm} components, {nnz} coupling non-zeros")
    o(f"struct PB3_{tag} {{ static constexpr int L = {L}, NP = {len(paths)}, NB = {lay3.nm}, NB2 = {lay2.nm}, D = {D}; }};")
    o(f"static const int pb3_{tag}_k[{len(outs)}] = {{{', '.join(str(lay3.k[l]) for l in outs)}}};")
    o(f"static const int pb3_{tag}_base[{len(outs)}] = {{{', '.join(str(lay3.base[l]) for l in outs)}}};")
    Ks = [w3j(slots[s][2], lb, l3) * math.sqrt(2 * l3 + 1) for s, lb, l3 in paths]
    o(f"struct PB3X_{tag} : PB3_{tag} {{")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void fwd(const T (&a)[{D}], const T (&b2)[{lay2.nm}], T* __restrict__ b3, long long stride) {{")
    for p, (s, lb, l3) in enumerate(paths):
        K, l1 = Ks[p], slots[s][2]
        for m3 in range(2 * l3 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * b2[{lay2.idx(s, m1)}] * a[{lb * lb + m2}]"
                     for m1 in range(2 * l1 + 1) for m2 in range(2 * lb + 1) if K[m1, m2, m3] != 0.0]
            o(f"    b3[{lay3.idx(p, m3)} * stride] = {' + '.join(terms) if terms else 'T(0)'};")
    o("  }")
    # gradient with respect to the second-order basis (accumulated into db2)
    o(f"  template <typename T> static TACE_HD TACE_INLINE void bwd_b2(const T (&a)[{D}], const T* __restrict__ db3, long long stride, T (&db2)[{lay2.nm}]) {{")
    for p, (s, lb, l3) in enumerate(paths):
        K, l1 = Ks[p], slots[s][2]
        o("    {")
        for m3 in range(2 * l3 + 1):
            o(f"      const T g{m3} = db3[{lay3.idx(p, m3)} * stride];")
        for m1 in range(2 * l1 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * a[{lb * lb + m2}] * g{m3}"
                     for m2 in range(2 * lb + 1) for m3 in range(2 * l3 + 1) if K[m1, m2, m3] != 0.0]
            if terms:
                o(f"      db2[{lay2.idx(s, m1)}] += {' + '.join(terms)};")
        o("    }")
    o("  }")
    # gradient with respect to A as the second operand (accumulated into da)
    o(f"  template <typename T> static TACE_HD TACE_INLINE void bwd_a(const T (&b2)[{lay2.nm}], const T* __restrict__ db3, long long stride, T (&da)[{D}]) {{")
    for p, (s, lb, l3) in enumerate(paths):
        K, l1 = Ks[p], slots[s][2]
        o("    {")
        for m3 in range(2 * l3 + 1):
            o(f"      const T g{m3} = db3[{lay3.idx(p, m3)} * stride];")
        for m2 in range(2 * lb + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * b2[{lay2.idx(s, m1)}] * g{m3}"
                     for m1 in range(2 * l1 + 1) for m3 in range(2 * l3 + 1) if K[m1, m2, m3] != 0.0]
            if terms:
                o(f"      da[{lb * lb + m2}] += {' + '.join(terms)};")
        o("    }")
    o("  }")
    o("};")
    return dict(tag="3:" + tag, P=len(paths), nb=lay3.nm, nnz=nnz)


def generate():
    """Text of ``tp_gen.cuh`` and one summary dictionary per generated struct."""
    out = [
        "// GENERATED by tace_b200/csrc/gen_tables.py -- do not edit by hand.",
        "// Path tables and unrolled contraction code for the interaction tensor product and the",
        "// product basis, ranks up to L = 3, natural-parity paths only.",
        "#pragma once",
        '#include "tace_common.cuh"',
        "namespace tace {",
    ]
    summary = []
    for L in (1, 2, 3):
        # source / output rank below the edge rank (the reference default is Lmax = 2, lmax = 3), then equal to it
        for Lin in [-1] + list(range(1, L + 1)):
            summary.append(gen_interaction(L, Lin, out))
        for Lout in [-1] + list(range(1, L + 1)):
            summary.append(gen_product(L, Lout, out))
        for Lout in [-1] + list(range(1, L + 1)):
            summary.append(gen_product3(L, Lout, out))
        for Lout in [-1] + list(range(1, L + 1)):
            summary.append(gen_product_bilinear(L, Lout, out))
    # coupling tables of the Wigner-matrix recursion D^l = (2l+1) C^T (D^1 (x) D^(l-1)) C (tace/models/o2/wigner.py:316-357)
    for l in (2, 3):
        c = w3j(1, l - 1, l)
        vals = ", ".join(repr(float(v)) for v in c.reshape(-1))
        out.append(f"// wigner_3j(1, {l - 1}, {l}), [3][{2 * l - 1}][{2 * l + 1}]")
        out.append(f"TACE_CONST double w3j_1_{l - 1}_{l}[{c.size}] = {{{vals}}};")
    out.append("}  // namespace tace")
    return "\n".join(out) + "\n", summary


def main():
    text, summary = generate()
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "tp_gen.cuh"), "w") as fh:
        fh.write(text)
    for s in summary:
        print(s)


if __name__ == "__main__":
    main()
