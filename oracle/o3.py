"""Restatement of the e3nn conventions the reference relies on.  TEST INFRASTRUCTURE ONLY.

e3nn is a third-party, unpinned dependency of the reference
(``pyproject.toml:21``) that is absent from the reference tree, so the
arithmetic below follows e3nn's published algorithms:

* real Wigner-3j symbols = SU(2) Clebsch-Gordan coefficients (Racah formula)
  conjugated into the real basis by ``Q_l`` and normalised to unit Frobenius
  norm (call sites ``tace/models/ictd.py:15,29,45``,
  ``tace/models/_e3nn/fused.py:44,116,203`` via ``o3.TensorProduct``);
* real spherical harmonics with ``y`` as the polar axis, component order
  ``m = -l..l`` (call site ``tace/models/angular.py:288-315``);
* ``normalize2mom`` second-moment constants (``tace/models/mlp.py:16-27``).

PARITY UNPINNED: no reference test pins 3j or spherical-harmonic values.
"""

from __future__ import annotations

import functools
import math
from fractions import Fraction
from math import factorial
from typing import List, Sequence, Tuple

import numpy as np
import torch


# ----------------------------------------------------------------------------
# Irreps bookkeeping (natural parity only: the parity of rank l is (-1)^l, the
# reference runs this path with ``parity=False``, ``_e3nn/base.py:16-30``).
# ----------------------------------------------------------------------------
class Irreps(list):
    """A list of ``(mul, l)`` blocks in e3nn ``mul_ir`` layout (m fastest)."""

    def __init__(self, items: Sequence[Tuple[int, int]] = ()):
        super().__init__((int(m), int(l)) for m, l in items)

    @property
    def dim(self) -> int:
        return sum(m * (2 * l + 1) for m, l in self)

    @property
    def lmax(self) -> int:
        return max(l for _, l in self)

    @property
    def ls(self) -> List[int]:
        return [l for _, l in self]

    def slices(self) -> List[slice]:
        out, acc = [], 0
        for m, l in self:
            out.append(slice(acc, acc + m * (2 * l + 1)))
            acc += m * (2 * l + 1)
        return out

    def simplify(self) -> "Irreps":
        out: List[Tuple[int, int]] = []
        for m, l in self:
            if out and out[-1][1] == l:
                out[-1] = (out[-1][0] + m, l)
            elif m > 0:
                out.append((m, l))
        return Irreps(out)

    def sort(self) -> "Irreps":
        return Irreps(sorted(self, key=lambda ml: ml[1]))  # stable in l

    def regroup(self) -> "Irreps":
        return self.sort().simplify()

    def __mul__(self, n: int) -> "Irreps":  # list repetition, as in e3nn
        return Irreps(list(self) * n)

    def __add__(self, other) -> "Irreps":
        return Irreps(list(self) + list(other))

    def __repr__(self) -> str:
        return "+".join(f"{m}x{l}{'e' if l % 2 == 0 else 'o'}" for m, l in self)

    @staticmethod
    def spherical_harmonics(lmax: int) -> "Irreps":
        return Irreps([(1, l) for l in range(lmax + 1)])


# ----------------------------------------------------------------------------
# Wigner 3j in the real basis
# ----------------------------------------------------------------------------
def _su2_cg_coeff(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> float:
    """<j1 m1 j2 m2 | j3 m3>, Condon-Shortley phase, Racah's closed form."""
    if m3 != m1 + m2:
        return 0.0
    vmin = max(-j1 + j2 + m3, -j1 + m1, 0)
    vmax = min(j2 + j3 + m1, j3 - j1 + j2, j3 + m3)
    f = factorial
    c = (2.0 * j3 + 1.0) * Fraction(
        f(j3 + j1 - j2) * f(j3 - j1 + j2) * f(j1 + j2 - j3) * f(j3 + m3) * f(j3 - m3),
        f(j1 + j2 + j3 + 1) * f(j1 - m1) * f(j1 + m1) * f(j2 - m2) * f(j2 + m2),
    )
    c = float(c) ** 0.5
    s = Fraction(0)
    for v in range(vmin, vmax + 1):
        s += (-1) ** (v + j2 + m2) * Fraction(
            f(j2 + j3 + m1 - v) * f(j1 - m1 + v),
            f(v) * f(j3 - j1 + j2 - v) * f(j3 + m3 - v) * f(v + j1 - j2 - m3),
        )
    return c * float(s)


def su2_clebsch_gordan(j1: int, j2: int, j3: int) -> np.ndarray:
    out = np.zeros((2 * j1 + 1, 2 * j2 + 1, 2 * j3 + 1))
    for m1 in range(-j1, j1 + 1):
        for m2 in range(-j2, j2 + 1):
            m3 = m1 + m2
            if abs(m3) <= j3:
                out[j1 + m1, j2 + m2, j3 + m3] = _su2_cg_coeff(j1, m1, j2, m2, j3, m3)
    return out


def change_basis_real_to_complex(l: int) -> np.ndarray:
    """Q_l with complex = Q real, including the (-i)^l factor that makes the
    conjugated Clebsch-Gordan coefficients real."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    for m in range(-l, 0):
        q[l + m, l + abs(m)] = 1 / 2**0.5
        q[l + m, l - abs(m)] = -1j / 2**0.5
    q[l, l] = 1
    for m in range(1, l + 1):
        q[l + m, l + abs(m)] = (-1) ** m / 2**0.5
        q[l + m, l - abs(m)] = 1j * (-1) ** m / 2**0.5
    return (-1j) ** l * q


@functools.lru_cache(maxsize=None)
def _wigner_3j_np(l1: int, l2: int, l3: int) -> np.ndarray:
    assert abs(l2 - l3) <= l1 <= l2 + l3
    q1 = change_basis_real_to_complex(l1)
    q2 = change_basis_real_to_complex(l2)
    q3 = change_basis_real_to_complex(l3)
    c = su2_clebsch_gordan(l1, l2, l3).astype(np.complex128)
    c = np.einsum("ij,kl,mn,ikn->jlm", q1, q2, np.conj(q3.T), c)
    assert np.abs(c.imag).max() < 1e-9
    c = c.real
    return c / np.linalg.norm(c)


def wigner_3j(l1: int, l2: int, l3: int, dtype=torch.float64) -> torch.Tensor:
    return torch.from_numpy(_wigner_3j_np(l1, l2, l3).copy()).to(dtype)


# ----------------------------------------------------------------------------
# Real spherical harmonics, polar axis y, ||Y_l||^2 = 1 on the unit sphere
# before the normalisation factor; "component" multiplies block l by sqrt(2l+1).
# ----------------------------------------------------------------------------
def spherical_harmonics(lmax: int, vec: torch.Tensor, normalization: str = "component") -> torch.Tensor:
    """Polynomials of the (already normalised, ``normalize=False``) edge vector.

    Returns ``[..., (lmax+1)^2]`` with blocks l = 0..lmax, m = -l..l.
    """
    if lmax > 3:
        raise NotImplementedError("oracle spherical harmonics are restated up to l = 3")
    x, y, z = vec[..., 0], vec[..., 1], vec[..., 2]
    out = [torch.ones_like(x)]
    if lmax >= 1:
        out += [x, y, z]
    if lmax >= 2:
        y2 = y * y
        x2z2 = x * x + z * z
        s20 = math.sqrt(3.0) * x * z
        s21 = math.sqrt(3.0) * x * y
        s22 = y2 - 0.5 * x2z2
        s23 = math.sqrt(3.0) * y * z
        s24 = math.sqrt(3.0) / 2.0 * (z * z - x * x)
        out += [s20, s21, s22, s23, s24]
    if lmax >= 3:
        s30 = math.sqrt(30.0) / 6.0 * (s20 * z + s24 * x)
        s31 = math.sqrt(5.0) * s20 * y
        s32 = math.sqrt(6.0) / 4.0 * (4.0 * y2 - x2z2) * x
        s33 = 0.5 * y * (2.0 * y2 - 3.0 * x2z2)
        s34 = math.sqrt(6.0) / 4.0 * z * (4.0 * y2 - x2z2)
        s35 = math.sqrt(5.0) * s24 * y
        s36 = math.sqrt(30.0) / 6.0 * (s24 * z - s20 * x)
        out += [s30, s31, s32, s33, s34, s35, s36]
    sh = torch.stack(out, dim=-1)
    if normalization == "component":
        scale = torch.cat(
            [torch.full((2 * l + 1,), math.sqrt(2 * l + 1), dtype=vec.dtype) for l in range(lmax + 1)]
        ).to(vec.device)
        sh = sh * scale
    elif normalization != "norm":
        raise ValueError(normalization)
    return sh


# ----------------------------------------------------------------------------
# normalize2mom: 1/sqrt(E[f(z)^2]), z ~ N(0,1), 10^6 seeded fp64 samples
# (tace/models/mlp.py:16-27 restates the same estimator).
# ----------------------------------------------------------------------------
@functools.lru_cache(maxsize=None)
def second_moment_constant(name: str) -> float:
    fn = {"silu": torch.nn.functional.silu, "sigmoid": torch.sigmoid, "tanh": torch.tanh}[name]
    gen = torch.Generator(device="cpu").manual_seed(0)
    z = torch.randn(1_000_000, generator=gen, dtype=torch.float64, device="cpu")
    return fn(z).square().mean().rsqrt().item()
