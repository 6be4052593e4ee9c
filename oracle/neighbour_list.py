"""Brute-force periodic neighbour list.  TEST INFRASTRUCTURE ONLY.

Restates the semantics the reference obtains from
``matscipy.neighbours.neighbour_list("ijSd")`` followed by its own filtering
(``tace/dataset/neighbour_list.py:240-247,284-298``): a full list (both
directions), ``D = r_j - r_i + S @ cell`` with strict ``|D| < cutoff`` in fp64,
self edges kept unless the shift is zero, shifts along non-periodic axes zero.
Row 0 of ``edge_index`` is ``i``, row 1 is ``j``.

matscipy (``pyproject.toml:18``, unpinned) is absent from the reference tree,
so this enumerates every periodic image explicitly instead of binning: parity
unpinned on degenerate geometries (a pair at exactly the cutoff).
"""

from __future__ import annotations

import numpy as np


def neighbour_list(positions: np.ndarray, cell: np.ndarray, pbc, cutoff: float):
    """Returns ``edge_index int64[2,E]``, ``edge_shifts int64[E,3]`` sorted by (i, j, S)."""
    pos = np.asarray(positions, dtype=np.float64)
    cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
    pbc = [bool(p) for p in pbc]
    n = pos.shape[0]
    if n == 0:
        return np.zeros((2, 0), np.int64), np.zeros((0, 3), np.int64)
    rng = [0, 0, 0]
    if any(pbc):
        vol = abs(np.linalg.det(cell))
        inv = np.linalg.inv(cell)
        frac = pos @ inv
        spread = frac.max(axis=0) - frac.min(axis=0)
        for k in range(3):
            if pbc[k]:
                a, b = cell[(k + 1) % 3], cell[(k + 2) % 3]
                height = vol / np.linalg.norm(np.cross(a, b))
                rng[k] = int(np.ceil(cutoff / height + spread[k])) + 1
    sx, sy, sz = np.meshgrid(*[np.arange(-r, r + 1) for r in rng], indexing="ij")
    shifts = np.stack([sx.ravel(), sy.ravel(), sz.ravel()], axis=1).astype(np.int64)
    c2 = cutoff * cutoff
    out_i, out_j, out_s = [], [], []
    for i in range(n):
        base = pos - pos[i]  # r_j - r_i, [n, 3]
        for s in shifts:
            t0 = s[0] * cell[0, 0] + s[1] * cell[1, 0] + s[2] * cell[2, 0]
            t1 = s[0] * cell[0, 1] + s[1] * cell[1, 1] + s[2] * cell[2, 1]
            t2 = s[0] * cell[0, 2] + s[1] * cell[1, 2] + s[2] * cell[2, 2]
            dx, dy, dz = base[:, 0] + t0, base[:, 1] + t1, base[:, 2] + t2
            d2 = dx * dx + dy * dy + dz * dz
            hit = d2 < c2
            if not s.any():
                hit[i] = False
            js = np.nonzero(hit)[0]
            if js.size:
                out_i.append(np.full(js.size, i, np.int64))
                out_j.append(js.astype(np.int64))
                out_s.append(np.broadcast_to(s, (js.size, 3)).copy())
    if not out_i:
        return np.zeros((2, 0), np.int64), np.zeros((0, 3), np.int64)
    i = np.concatenate(out_i)
    j = np.concatenate(out_j)
    s = np.concatenate(out_s)
    order = np.lexsort((s[:, 2], s[:, 1], s[:, 0], j, i))
    return np.stack([i[order], j[order]]), s[order]


def canonical_sort(edge_index: np.ndarray, edge_shifts: np.ndarray):
    """Sort an edge list by (i, j, Sx, Sy, Sz) so two lists can be compared bit for bit."""
    ei = np.asarray(edge_index, dtype=np.int64)
    es = np.asarray(edge_shifts).astype(np.int64)
    order = np.lexsort((es[:, 2], es[:, 1], es[:, 0], ei[1], ei[0]))
    return ei[:, order], es[order]
