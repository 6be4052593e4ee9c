"""Neighbour lists on the GPU behind the reference's ``get_neighborhood`` interface
(``tace/dataset/neighbour_list.py:195-298``).

``neighbor_list_batch`` is the device-resident form (one call for a whole batch of
structures); ``get_neighborhood`` keeps the reference signature and numpy return types.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple, Union

import numpy as np
import torch

from . import lib as _lib


def complete_cell(lattice: np.ndarray, positions: np.ndarray, pbc, cutoff: float) -> np.ndarray:
    """Replace missing (zero) cell vectors along non-periodic axes by vectors orthogonal to the
    others and long enough to hold the structure, so the cell is invertible (the reference calls
    ``ase.geometry.complete_cell`` for the same purpose, tace/dataset/neighbour_list.py:237)."""
    cell = np.array(lattice, dtype=np.float64).reshape(3, 3).copy()
    extent = float(np.ptp(positions, axis=0).max()) if len(positions) else 1.0
    length = extent + 2.0 * cutoff + 1.0
    missing = [k for k in range(3) if np.allclose(cell[k], 0.0)]
    if any(pbc[k] for k in missing):
        raise ValueError("At least one direction is periodic, but lattice is None or zero.")
    present = [k for k in range(3) if k not in missing]
    for k in missing:
        if len(present) == 2:
            v = np.cross(cell[present[0]], cell[present[1]])
        elif len(present) == 1:
            a = cell[present[0]]
            trial = np.eye(3)[int(np.argmin(np.abs(a)))]
            v = np.cross(a, trial)
        else:
            v = np.eye(3)[k]
        cell[k] = v / np.linalg.norm(v) * length
        present.append(k)
    if np.linalg.det(cell) < 0 and missing:
        cell[missing[0]] *= -1.0
    return cell


def neighbor_list_batch(positions: torch.Tensor, lattice: torch.Tensor, pbc: torch.Tensor, graph_ptr: torch.Tensor,
                        cutoff: float, n_targets: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """positions fp64 [N,3], lattice fp64 [B,3,3], pbc uint8 [B,3], graph_ptr int32 [B+1], all on
    one CUDA device.  Returns ``edge_index int64[2,E]`` (row 0 = source, row 1 = target, grouped by
    target) and ``edge_shifts int32[E,3]`` with edge vector = r[target] - r[source] + shift @ cell.
    ``n_targets``: keep only edges whose target is one of the first ``n_targets`` atoms (the owned
    atoms of a domain; the rest are ghost copies that only act as sources)."""
    lib = _lib.load()
    dev = positions.device
    if dev.type != "cuda":
        raise _lib.TaceError("tace_b200 neighbour lists run on CUDA devices only")
    positions = positions.to(torch.float64).contiguous()
    lattice = lattice.to(torch.float64).reshape(-1, 3, 3).contiguous()
    pbc = pbc.to(torch.uint8).reshape(-1, 3).contiguous()
    graph_ptr = graph_ptr.to(torch.int32).contiguous()
    n, b = positions.shape[0], lattice.shape[0]
    counts = torch.zeros(n, dtype=torch.int32, device=dev)
    need = ctypes.c_size_t()
    _lib.check(lib.tace_nl_workspace_bytes(n, b, ctypes.byref(need)), "tace_nl_workspace_bytes")
    work = torch.empty(int(need.value), dtype=torch.uint8, device=dev)  # torch's caching allocator: no cudaMalloc once warm
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(lib.tace_nl_count(positions.data_ptr(), lattice.data_ptr(), pbc.data_ptr(), graph_ptr.data_ptr(), b, n,
                                     float(cutoff), counts.data_ptr(), work.data_ptr(), work.numel(), stream), "tace_nl_count")
        if n_targets is not None and n_targets < n:
            counts[n_targets:] = 0  # rows without edges start at the end of the list and write nothing
        row_ptr = torch.zeros(n + 1, dtype=torch.int64, device=dev)
        torch.cumsum(counts, 0, out=row_ptr[1:])
        n_edges = int(row_ptr[-1].item())
        edge_index = torch.empty(2, n_edges, dtype=torch.int64, device=dev)
        shifts = torch.empty(n_edges, 3, dtype=torch.int32, device=dev)
        _lib.check(lib.tace_nl_fill(positions.data_ptr(), lattice.data_ptr(), pbc.data_ptr(), graph_ptr.data_ptr(), b, n,
                                    float(cutoff), row_ptr.data_ptr(), n_edges, edge_index.data_ptr(), shifts.data_ptr(),
                                    work.data_ptr(), work.numel(), stream), "tace_nl_fill")
    return edge_index, shifts


def get_neighborhood(positions: np.ndarray, cutoff: float, pbc: Union[bool, Tuple[bool, bool, bool], None] = None,
                     lattice: Optional[np.ndarray] = None, max_neighbors: Optional[int] = None, backend: str = "tace_b200",
                     device: Union[str, torch.device] = "cuda"):
    """Reference signature and return value: ``(edge_index[2,E], edge_shifts[E,3], pbc, lattice)`` as numpy."""
    if pbc is None:
        pbc = (False, False, False)
    elif isinstance(pbc, bool):
        pbc = (pbc,) * 3
    else:
        pbc = tuple(bool(i) for i in pbc)
    if len(pbc) != 3:
        raise ValueError(f"pbc must contain three values, got {pbc}")
    positions = np.asarray(positions)
    if lattice is None:
        lattice = np.zeros((3, 3), dtype=positions.dtype)
    else:
        lattice = np.asarray(lattice, dtype=positions.dtype)
        if lattice.shape != (3, 3):
            raise ValueError(f"lattice must have shape (3, 3), got {lattice.shape}")
        lattice = lattice.copy()
    if any(pbc) and np.allclose(lattice, 0.0):
        raise ValueError("At least one direction is periodic, but lattice is None or zero.")
    cell = complete_cell(lattice, positions, pbc, cutoff)
    dev = torch.device(device)
    ei, es = neighbor_list_batch(
        torch.as_tensor(positions, dtype=torch.float64, device=dev), torch.as_tensor(cell, device=dev)[None],
        torch.tensor([pbc], dtype=torch.uint8, device=dev), torch.tensor([0, len(positions)], dtype=torch.int32, device=dev),
        cutoff)
    return ei.cpu().numpy(), es.cpu().numpy().astype(np.int64), pbc, lattice
