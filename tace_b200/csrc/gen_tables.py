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
def gen_interaction(L, scalar_src, out):
    tag = f"L{L}_{'S' if scalar_src else 'F'}"
    in1 = [0] if scalar_src else list(range(L + 1))
    sh = list(range(L + 1))
    outs = list(range(L + 1))
    paths = tp_paths(L, in1, sh, outs)
    lay = Layout(paths, outs)
    xoff = {l: (0 if scalar_src else l * l) for l in in1}
    nx = 1 if scalar_src else (L + 1) ** 2
    D = (L + 1) ** 2
    # G holds, per edge, only the structurally non-zero entries of
    # G^p[m1][m3] = sum_m2 K^p[m1,m2,m3] * Y[l2^2 + m2]; gi[(p, m1, m3)] is the compact index.
    gi, g_start, g_y, g_c = {}, [0], [], []
    nnz_total = 0
    for p, (l1, l2, l3) in enumerate(paths):
        K = w3j(l1, l2, l3) * math.sqrt(2 * l3 + 1)
        nnz_total += int(np.count_nonzero(K))
        for m1 in range(2 * l1 + 1):
            for m3 in range(2 * l3 + 1):
                m2s = [m2 for m2 in range(2 * l2 + 1) if K[m1, m2, m3] != 0.0]
                if not m2s:
                    continue
                gi[(p, m1, m3)] = len(g_start) - 1
                for m2 in m2s:
                    g_y.append(l2 * l2 + m2)
                    g_c.append(K[m1, m2, m3])
                g_start.append(len(g_y))
    ng = len(g_start) - 1
    P = len(paths)

    o = out.append
    o(f"// ---- interaction tensor product, L={L}, {'scalar' if scalar_src else 'full'} source: "
      f"{P} paths, {lay.nm} message components, {ng} non-zero G entries, {nnz_total} coupling non-zeros")
    o(f"struct TP_{tag} {{")
    o(f"  static constexpr int L = {L}, NP = {P}, NX = {nx}, NM = {lay.nm}, NG = {ng}, D = {D}, NNZ = {len(g_y)};")
    o("};")
    o(f"static const int tp_{tag}_path_l3[{P}] = {{{', '.join(str(p[2]) for p in paths)}}};")
    o(f"static const int tp_{tag}_k[{L + 1}] = {{{', '.join(str(lay.k[l]) for l in outs)}}};")
    o(f"static const int tp_{tag}_base[{L + 1}] = {{{', '.join(str(lay.base[l]) for l in outs)}}};")
    o(f"static const int tp_{tag}_plocal[{P}] = {{{', '.join(str(v) for v in lay.plocal)}}};")
    o(f"TACE_CONST short tp_{tag}_gstart[{ng + 1}] = {{{', '.join(str(v) for v in g_start)}}};")
    o(f"TACE_CONST unsigned char tp_{tag}_gy[{len(g_y)}] = {{{', '.join(str(v) for v in g_y)}}};")
    o(f"TACE_CONST double tp_{tag}_gc[{len(g_c)}] = {{{', '.join(repr(float(v)) for v in g_c)}}};")

    def gterm(p, m1, m3):
        return gi.get((p, m1, m3))

    # forward: acc[idx(p,m3)] += w[p] * sum_m1 x[m1] G[m1][m3]
    o("template <typename T>")
    o(f"TACE_HD TACE_INLINE void tp_fwd_{tag}(const T (&x)[{nx}], const T* __restrict__ G, const T (&w)[{P}], T (&acc)[{lay.nm}]) {{")
    for p, (l1, l2, l3) in enumerate(paths):
        for m3 in range(2 * l3 + 1):
            terms = [f"x[{xoff[l1] + m1}] * G[{gterm(p, m1, m3)}]" for m1 in range(2 * l1 + 1)
                     if gterm(p, m1, m3) is not None]
            if terms:
                o(f"  acc[{lay.idx(p, m3)}] += w[{p}] * ({' + '.join(terms)});")
    o("}")

    # backward wrt x (source features): dx[m1] += w[p] * sum_m3 G[m1][m3] g[idx(p,m3)]
    o("template <typename T>")
    o(f"TACE_HD TACE_INLINE void tp_bwdx_{tag}(const T (&g)[{lay.nm}], const T* __restrict__ G, const T (&w)[{P}], T (&dx)[{nx}]) {{")
    for p, (l1, l2, l3) in enumerate(paths):
        for m1 in range(2 * l1 + 1):
            terms = [f"G[{gterm(p, m1, m3)}] * g[{lay.idx(p, m3)}]" for m3 in range(2 * l3 + 1)
                     if gterm(p, m1, m3) is not None]
            if terms:
                o(f"  dx[{xoff[l1] + m1}] += w[{p}] * ({' + '.join(terms)});")
    o("}")

    # backward wrt per-edge weights and angular features
    o("template <typename T>")
    o(f"TACE_HD TACE_INLINE void tp_bwdw_{tag}(const T (&x)[{nx}], const T (&g)[{lay.nm}], const T* __restrict__ G, "
      f"const T (&w)[{P}], T (&dw)[{P}], T (&dY)[{D}]) {{")
    for p, (l1, l2, l3) in enumerate(paths):
        n3 = 2 * l3 + 1
        K = w3j(l1, l2, l3) * math.sqrt(2 * l3 + 1)
        o("  {")
        pairs = [(m1, m3) for m1 in range(2 * l1 + 1) for m3 in range(n3) if gterm(p, m1, m3) is not None]
        for m1, m3 in pairs:
            o(f"    const T q{m1}_{m3} = x[{xoff[l1] + m1}] * g[{lay.idx(p, m3)}];")
        terms = [f"G[{gterm(p, m1, m3)}] * q{m1}_{m3}" for m1, m3 in pairs]
        o(f"    dw[{p}] = {' + '.join(terms)};")
        for m2 in range(2 * l2 + 1):
            terms = [f"{lit(float(K[m1, m2, m3]))} * q{m1}_{m3}"
                     for m1, m3 in pairs if K[m1, m2, m3] != 0.0]
            if terms:
                o(f"    dY[{l2 * l2 + m2}] += w[{p}] * ({' + '.join(terms)});")
        o("  }")
    o("}")
    o(f"struct TPX_{tag} : TP_{tag} {{")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void fwd(const T (&x)[{nx}], const T* __restrict__ G, const T (&w)[{P}], "
      f"T (&acc)[{lay.nm}]) {{ tp_fwd_{tag}<T>(x, G, w, acc); }}")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void bwdx(const T (&g)[{lay.nm}], const T* __restrict__ G, const T (&w)[{P}], "
      f"T (&dx)[{nx}]) {{ tp_bwdx_{tag}<T>(g, G, w, dx); }}")
    o(f"  template <typename T> static TACE_HD TACE_INLINE void bwdw(const T (&x)[{nx}], const T (&g)[{lay.nm}], const T* __restrict__ G, "
      f"const T (&w)[{P}], T (&dw)[{P}], T (&dY)[{D}]) {{ tp_bwdw_{tag}<T>(x, g, G, w, dw, dY); }}")
    o(f"  static TACE_D TACE_INLINE const short* gstart() {{ return tp_{tag}_gstart; }}")
    o(f"  static TACE_D TACE_INLINE const unsigned char* gy() {{ return tp_{tag}_gy; }}")
    o(f"  static TACE_D TACE_INLINE const double* gc() {{ return tp_{tag}_gc; }}")
    o("};")
    return dict(tag=tag, P=P, nm=lay.nm, ng=ng, nnz=nnz_total)


# ------------------------------------------------------------- product basis code
def gen_product(L, last, out):
    tag = f"L{L}_{'T' if last else 'A'}"  # T = target (scalar) outputs only, A = all ranks
    ls = list(range(L + 1))
    outs = [0] if last else ls
    paths = tp_paths(L, ls, ls, outs)
    lay = Layout(paths, outs)
    D = (L + 1) ** 2
    P = len(paths)
    o = out.append
    nnz = sum(int(np.count_nonzero(w3j(*p))) for p in paths)
    o(f"// ---- product basis (A x A), L={L}, {'scalar outputs' if last else 'all ranks'}: {P} paths, "
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


def main():
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
        for scalar_src in (True, False):
            summary.append(gen_interaction(L, scalar_src, out))
        for last in (False, True):
            summary.append(gen_product(L, last, out))
    out.append("}  // namespace tace")
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "tp_gen.cuh"), "w") as fh:
        fh.write("\n".join(out) + "\n")
    for s in summary:
        print(s)


if __name__ == "__main__":
    main()
